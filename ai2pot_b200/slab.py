"""Spatial decomposition of one large periodic system into slabs along the first lattice vector,
one slab per rank / GPU, for energy + force + virial evaluation.

This is the role LAMMPS plays for the reference (`interface/lammps/AI2POT/pair_ai2pot.cpp:177-205,
452-455`: the pair style evaluates local + ghost atoms and returns forces on both; LAMMPS
exchanges ghost positions before and reverse-communicates ghost forces after). Here:

  set-up   each rank keeps the atoms whose fractional coordinate along a0 lies in its slab, ordered
           [interior | boundary]: boundary atoms lie within the halo width of a slab face (they are
           what the face neighbours need as ghosts, and the only centres that can see a ghost)
  step     1. halo exchange: boundary positions to the two face neighbours (periodic; the wrapped
              copies are shifted by -/+ a0 with the reference's own image arithmetic r + a0*n)
           2. neighbour rows + model evaluation, in passes over disjoint ranges of centres
           3. ghost forces go back to their owners and are added ("ghost-force reduction")
           4. all-reduce of the energy and the nine virial components

Three schedules of a step (`SlabStep`):
  "serial"   1 -> 2 (one pass over all owned centres) -> 3 -> 4, one stream
  "overlap"  interior centres need no ghost, so a first pass over part of them runs while the halo
             is in flight on a second stream; then the boundary pass; then the rest of the interior
             while the ghost forces travel back
  "owner"    owner-computes variant: the halo is twice the cutoff wide and the ghosts within one
             cutoff of the face are evaluated as centres too (forces only), so every force on an
             owned atom is computed locally and step 3 disappears

`torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the messages; message sizes are
fixed at set-up, so a step makes no host synchronisation. With `transport="peer"` the two neighbour
exchanges of a step are this library's own kernels instead: the boundary rows are gathered, shifted and
stored straight into the neighbour GPU's arrays over NVLink (`ai2b_peer_push_rows_*`, arrays in
`torch.distributed._symmetric_memory`), a flag follows the data, and the receiving stream is held by a
bounded wait (`ai2b_peer_wait`); only the all-reduce of energy and virial stays with NCCL. The per-pass compute is injected
(`CudaPasses` on a GPU), so the partition / exchange / schedule logic is tested on CPU ranks.

Positions of the owned atoms may be updated in place between steps (`SlabDomain.owned`), as an MD
host does, as long as no atom moves more than half the `skin` the domain was built with:
ownership, send lists and the interior/boundary split are fixed at set-up. `SlabStep.check_status()`
verifies that (and the neighbour-row overflow flag); beyond it, build a new `SlabDomain`.
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
    def __init__(self, cell, coords, types, rcut, rank, nranks, device, dist=None, halo_margin=1e-6, skin=0.0, halo_cutoffs=1,
                 transport="nccl"):
        """cell [3,3], coords [N,3], types [N] describe the WHOLE system (host arrays, identical on
        every rank); each rank keeps only its slab. halo_cutoffs = 2 builds the wide halo of the
        owner-computes schedule."""
        self.rank, self.P, self.dist, self.device = rank, nranks, dist, device
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.transport = transport if nranks > 1 else "nccl"
        self.cell = np.asarray(cell)
        self.rcut, self.skin, self.halo_cutoffs = float(rcut), float(skin), int(halo_cutoffs)
        self.dtype = torch.float64 if np.asarray(coords).dtype == np.float64 else torch.float32
        a = np.asarray(cell, np.float64)
        n0 = np.cross(a[1], a[2])
        d0 = abs(a[0] @ (n0 / np.linalg.norm(n0)))          # slab-normal extent of the cell
        self.d0 = d0
        self.width = d0 / nranks
        reach = rcut + skin + halo_margin                    # how far a centre can see, with the motion allowance
        halo = self.halo_cutoffs * rcut + skin + halo_margin
        if nranks > 1 and self.width < halo:
            raise ValueError(f"slab width {self.width:.3f} is below the halo {halo:.3f} ({self.halo_cutoffs} x cutoff {rcut}): use fewer ranks")
        owner, fx, wrap = partition(cell, coords, nranks)
        mine = np.nonzero(owner == rank)[0]
        f = fx[mine] * nranks - rank                         # position inside the slab, [0,1)
        hs = halo / d0 * nranks                              # halo and reach in slab-width units
        rs = reach / d0 * nranks
        if nranks > 1:
            boundary = (f < rs) | (f >= 1.0 - rs)
            order = np.concatenate([np.nonzero(~boundary)[0], np.nonzero(boundary)[0]])   # [interior | boundary]
            mine, f = mine[order], f[order]
            self.n_interior = int((~boundary).sum())
        else:
            self.n_interior = len(mine)
        self.global_index = mine
        self.nlocal = len(mine)
        # positions are brought into the cell along a0 (the input may be unwrapped), so that a slab is contiguous
        inside = np.asarray(coords)[mine] - (wrap[mine, None] * np.asarray(cell)[0][None]).astype(np.asarray(coords).dtype)
        owned = torch.from_numpy(np.ascontiguousarray(inside)).to(device)
        self.owned_types = torch.from_numpy(np.ascontiguousarray(np.asarray(types)[mine], dtype=np.int32)).to(device)
        self.a0 = torch.from_numpy(np.ascontiguousarray(self.cell[0])).to(self.dtype).to(device)
        # send lists, one per (side, shell): shell 0 = within `reach` of the face (what a one-cutoff halo needs),
        # shell 1 = the rest of a wide halo. Ghost rows are laid out shell-major: [L0 | R0 | L1 | R1].
        if nranks == 1:
            sends = [np.zeros(0, np.int64)] * 4
        else:
            l0, r0 = f < rs, f >= 1.0 - rs
            if self.halo_cutoffs > 1:
                l1, r1 = (f < hs) & ~l0, (f >= 1.0 - hs) & ~r0
            else:
                l1 = r1 = np.zeros(len(f), bool)
            sends = [np.nonzero(m)[0] for m in (l0, r0, l1, r1)]
        self.send_lists = [torch.from_numpy(s).to(device) for s in sends]      # [to-left 0, to-right 0, to-left 1, to-right 1]
        self.left, self.right = (rank - 1) % nranks, (rank + 1) % nranks
        # ghost counts: what the neighbours send us
        counts = torch.tensor([len(s) for s in sends], dtype=torch.int64)
        if nranks > 1:
            allc = [torch.zeros(4, dtype=torch.int64) for _ in range(nranks)]
            self._all_gather_cpu(allc, counts)
            # from the left neighbour we get what it sends to ITS right, and vice versa
            self.recv_counts = [int(allc[self.left][1]), int(allc[self.right][0]), int(allc[self.left][3]), int(allc[self.right][2])]
        else:
            self.recv_counts = [0, 0, 0, 0]
        self.nghost = sum(self.recv_counts)
        self.n_inner_ghost = self.recv_counts[0] + self.recv_counts[1]       # ghosts within one cutoff of a face
        self.ntotal = self.nlocal + self.nghost
        # one buffer [owned | ghost L0 | ghost R0 | ghost L1 | ghost R1]; `owned` is a view of its head
        if self.transport == "peer":
            self._peer_setup_begin([len(s) for s in sends])
            self.local = self._sym_local[: self.ntotal * 3].view(self.ntotal, 3)
        else:
            self.local = torch.empty(self.ntotal, 3, dtype=self.dtype, device=device)
        self.local[: self.nlocal] = owned
        self.owned = self.local[: self.nlocal]
        self.owned_at_setup = self.owned.clone()
        off = np.concatenate([[self.nlocal], self.nlocal + np.cumsum(self.recv_counts)]).astype(int)
        self.ghost_slices = [slice(int(off[k]), int(off[k + 1])) for k in range(4)]   # rows of [from-left 0, from-right 0, from-left 1, from-right 1]
        self.ghost_views = [self.local[s] for s in self.ghost_slices]
        # ghost types travel once
        self.types = torch.empty(self.ntotal, dtype=torch.int32, device=device)
        self.types[: self.nlocal] = self.owned_types
        # Periodic wrap of the end slabs: copies going "around" the cell are shifted by -/+ a0. The sender
        # applies it, with the reference's image arithmetic r + a0 * n (source/nblist/include/structure.h:654-682).
        self.send_idx = torch.cat(self.send_lists)
        nsend = len(self.send_idx)
        soff = np.concatenate([[0], np.cumsum([len(s) for s in sends])]).astype(int)
        self.send_slices = [slice(int(soff[k]), int(soff[k + 1])) for k in range(4)]
        self.send_buf = torch.empty(nsend, 3, dtype=self.dtype, device=device)
        self.send_views = [self.send_buf[s] for s in self.send_slices]
        # ghost forces coming home (one-cutoff halo only): rows line up with send lists 0 and 1
        nback = len(sends[0]) + len(sends[1])
        self.back = self._sym_back[: nback * 3].view(nback, 3) if self.transport == "peer" else \
            torch.empty(nback, 3, dtype=self.dtype, device=device)
        self.back_idx = self.send_idx[:nback]
        shift = torch.zeros(nsend, 3, dtype=self.dtype, device=device)
        if nranks > 1 and rank == 0:                        # my left neighbour is the last slab: it sees these one cell up
            for k in (0, 2):
                shift[self.send_slices[k]] = self.a0 * 1.0
        if nranks > 1 and rank == nranks - 1:               # my right neighbour is slab 0
            for k in (1, 3):
                shift[self.send_slices[k]] = self.a0 * -1.0
        self.send_shift = shift if (nranks > 1 and (rank == 0 or rank == nranks - 1)) else None
        self.pbc = (nranks == 1, True, True)
        # fractional extent of the local atoms along a0 (with the halo and the motion allowance): lets the
        # neighbour build size its grid on the host instead of reducing over the positions every step
        lo = rank / nranks - (halo + skin) / d0
        hi = (rank + 1) / nranks + (halo + skin) / d0
        self.open_extent = None if nranks == 1 else (lo, hi)
        if self.transport == "peer":
            self._peer_setup_finish()
        if nranks > 1:
            tys = [self.owned_types[s].contiguous() for s in self.send_lists]
            got = self._exchange(tys, [torch.empty(c, dtype=torch.int32, device=device) for c in self.recv_counts])
            for s, t in zip(self.ghost_slices, got):
                self.types[s] = t

    # -- plumbing ----------------------------------------------------------------------------------
    def _all_gather_cpu(self, out, t):
        if self.dist.get_backend() == "nccl":
            dev = [o.to(self.device) for o in out]
            self.dist.all_gather(dev, t.to(self.device))
            for o, d in zip(out, dev):
                o.copy_(d.cpu())
        else:
            self.dist.all_gather(out, t)

    def _exchange(self, send, recv):
        """send = [to-left 0, to-right 0, to-left 1, to-right 1], recv = [from-left 0, from-right 0, from-left 1, from-right 1]
        (empty messages are skipped on both ends). Tag = 2 * shell + direction (0 towards lower x, 1 towards higher x).
        With two ranks both neighbours are the same peer; the tags (gloo) and the posting order (NCCL, which ignores
        tags: the k-th receive from a peer matches its k-th send) keep the messages apart: what the peer sent
        towards lower x arrives as our right-hand ghosts."""
        d = self.dist
        ops = []
        for shell in (0, 1):
            tl, tr = send[2 * shell], send[2 * shell + 1]
            fl, fr = recv[2 * shell], recv[2 * shell + 1]
            if tl.shape[0]:
                ops.append(d.P2POp(d.isend, tl, self.left, tag=2 * shell))
            if tr.shape[0]:
                ops.append(d.P2POp(d.isend, tr, self.right, tag=2 * shell + 1))
            if fr.shape[0]:
                ops.append(d.P2POp(d.irecv, fr, self.right, tag=2 * shell))
            if fl.shape[0]:
                ops.append(d.P2POp(d.irecv, fl, self.left, tag=2 * shell + 1))
        if ops:
            for r in d.batch_isend_irecv(ops):
                r.wait()
        return recv

    # -- peer transport: symmetric arrays, row maps, flags -------------------------------------------------
    def _peer_setup_begin(self, nsend):
        """Symmetric-memory arrays (same size on every rank) for the positions and the returning ghost forces, and the
        geometry of every rank (owned count, ghost counts, send counts) so that a rank knows where its rows land."""
        import torch.distributed._symmetric_memory as symm
        d = self.dist
        mine = torch.tensor([self.nlocal] + self.recv_counts + list(nsend), dtype=torch.int64)
        allg = [torch.zeros(9, dtype=torch.int64) for _ in range(self.P)]
        self._all_gather_cpu(allg, mine)
        self._geom = [[int(v) for v in g] for g in allg]           # per rank: nlocal, recv[4], nsend[4]
        max_total = max(g[0] + sum(g[1:5]) for g in self._geom)
        max_back = max(g[5] + g[6] for g in self._geom)
        self._sym_local = symm.empty(max(max_total, 1) * 3, dtype=self.dtype, device=self.device)
        self._sym_back = symm.empty(max(max_back, 1) * 3, dtype=self.dtype, device=self.device)
        # flags: [0..3] halo from left / right, forces from left / right; [8 + P h + q] partial sums of rank q have arrived
        # (h = step parity: tables and their flags are double-buffered, so a rank that is a step ahead never writes
        # into a table another rank is still summing)
        self._sym_flags = symm.empty(8 + 2 * self.P, dtype=torch.int32, device=self.device)
        self._sym_flags.zero_()
        self._sym_table = symm.empty(2 * self.P * 16, dtype=self.dtype, device=self.device)     # [parity][rank][16] partial energy / virial
        self._sym_table.zero_()
        group = d.group.WORLD
        self._h_local = symm.rendezvous(self._sym_local, group)
        self._h_back = symm.rendezvous(self._sym_back, group)
        self._h_flags = symm.rendezvous(self._sym_flags, group)
        self._h_table = symm.rendezvous(self._sym_table, group)
        self._max_total, self._max_back = max_total, max_back

    def _peer_setup_finish(self):
        """Row maps of the pushes. Ghost rows of a rank are laid out [from-left 0 | from-right 0 | from-left 1 | from-right 1]
        after its owned rows; what goes to the LEFT neighbour lands in its from-RIGHT rows and vice versa. Returning
        forces land in the owner's `back` rows, which follow its send lists 0 (to-left) and 1 (to-right)."""
        dev, i32 = self.device, torch.int32
        gl, gr = self._geom[self.left], self._geom[self.right]

        def ghost_off(g, k):            # first row of ghost slice k on a rank with geometry g
            return g[0] + sum(g[1:1 + k])
        peer_local = {p: self._h_local.get_buffer(p, (self._max_total * 3,), self.dtype) for p in {self.left, self.right}}
        peer_back = {p: self._h_back.get_buffer(p, (self._max_back * 3,), self.dtype) for p in {self.left, self.right}}
        peer_flags = {p: self._h_flags.get_buffer(p, (8 + 2 * self.P,), torch.int32) for p in {self.left, self.right}}
        # every rank's table and table flags, for the all-to-all of the partial energy / virial
        P = self.P
        self._all_tables = [self._sym_table if q == self.rank else self._h_table.get_buffer(q, (2 * P * 16,), self.dtype) for q in range(P)]
        self._all_flags = [self._sym_flags if q == self.rank else self._h_flags.get_buffer(q, (8 + 2 * P,), torch.int32) for q in range(P)]
        self._table_ptrs = [torch.tensor([t[h * P * 16:].data_ptr() for t in self._all_tables], dtype=torch.int64, device=dev) for h in (0, 1)]
        self._table_flag_ptrs = [torch.tensor([f[8 + h * P:].data_ptr() for f in self._all_flags], dtype=torch.int64, device=dev) for h in (0, 1)]
        self._back_idx32 = None
        # halo pushes: source rows = my send lists, destination rows in the neighbour's position array
        src_l = torch.cat([self.send_lists[0], self.send_lists[2]]).to(i32)
        dst_l = torch.cat([torch.arange(len(self.send_lists[0]), device=dev) + ghost_off(gl, 1),
                           torch.arange(len(self.send_lists[2]), device=dev) + ghost_off(gl, 3)]).to(i32)
        src_r = torch.cat([self.send_lists[1], self.send_lists[3]]).to(i32)
        dst_r = torch.cat([torch.arange(len(self.send_lists[1]), device=dev) + ghost_off(gr, 0),
                           torch.arange(len(self.send_lists[3]), device=dev) + ghost_off(gr, 2)]).to(i32)
        assert len(self.send_lists[0]) == gl[2] and len(self.send_lists[1]) == gr[1] and len(self.send_lists[2]) == gl[4] and \
            len(self.send_lists[3]) == gr[3], "neighbour ghost counts do not match the send lists"
        a0 = self.cell[0].astype(np.float64)
        self._push = dict(
            halo_left=dict(src_idx=src_l.contiguous(), dst_idx=dst_l.contiguous(), shift=(a0 if self.rank == 0 else None),
                           dst=peer_local[self.left], flag=peer_flags[self.left][1:2]),       # arrives as its from-right data
            halo_right=dict(src_idx=src_r.contiguous(), dst_idx=dst_r.contiguous(), shift=(-a0 if self.rank == self.P - 1 else None),
                            dst=peer_local[self.right], flag=peer_flags[self.right][0:1]),
            # ghost forces: my from-left ghost rows are the left neighbour's send list 1 -> its back rows after its list 0
            force_left=dict(src0=ghost_off(self._geom[self.rank], 0), n=self.recv_counts[0], dst0=gl[5], dst=peer_back[self.left],
                            flag=peer_flags[self.left][3:4]),
            force_right=dict(src0=ghost_off(self._geom[self.rank], 1), n=self.recv_counts[1], dst0=0, dst=peer_back[self.right],
                             flag=peer_flags[self.right][2:3]))
        assert self.recv_counts[0] == gl[6] and self.recv_counts[1] == gr[5]
        self._counter = torch.zeros(4, dtype=torch.int32, device=dev)
        self.peer_status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._epoch = 0
        self.dist.barrier()

    def _peer_halo_exchange(self):
        from . import capi
        self._epoch += 1
        pl, pr = self._push["halo_left"], self._push["halo_right"]
        capi.peer_exchange(dict(src=self.owned, src_idx=pl["src_idx"], dst_idx=pl["dst_idx"], n=len(pl["src_idx"]), shift=pl["shift"],
                                dst=pl["dst"], flag=pl["flag"]),
                           dict(src=self.owned, src_idx=pr["src_idx"], dst_idx=pr["dst_idx"], n=len(pr["src_idx"]), shift=pr["shift"],
                                dst=pr["dst"], flag=pr["flag"]),
                           self._epoch, self._sym_flags[0:1], self._sym_flags[1:2], self.peer_status, self._counter[0:1])

    def _peer_return_ghost_forces(self, force):
        from . import capi
        pl, pr = self._push["force_left"], self._push["force_right"]
        capi.peer_exchange(dict(src=force[pl["src0"]: pl["src0"] + pl["n"]], n=pl["n"], dst=pl["dst"][pl["dst0"] * 3:], flag=pl["flag"]),
                           dict(src=force[pr["src0"]: pr["src0"] + pr["n"]], n=pr["n"], dst=pr["dst"][pr["dst0"] * 3:], flag=pr["flag"]),
                           self._epoch, self._sym_flags[2:3], self._sym_flags[3:4], self.peer_status, self._counter[1:2])

    def peer_finish(self, force, partial, reduced, with_forces=True):
        """The closing exchange of a step in one launch (peer transport): ghost-force rows to the neighbours, partial
        energy / virial to every rank, received rows added onto the owned atoms, partials summed in rank order."""
        from . import capi
        pl, pr = self._push["force_left"], self._push["force_right"]
        if self._back_idx32 is None:
            self._back_idx32 = self.back_idx.to(torch.int32).contiguous()
        left = right = None
        if with_forces:
            left = dict(src=force[pl["src0"]: pl["src0"] + pl["n"]], n=pl["n"], dst=pl["dst"][pl["dst0"] * 3:], flag=pl["flag"])
            right = dict(src=force[pr["src0"]: pr["src0"] + pr["n"]], n=pr["n"], dst=pr["dst"][pr["dst0"] * 3:], flag=pr["flag"])
        h, P = self._epoch & 1, self.P
        capi.peer_return_reduce(left, right, self._epoch, self._sym_flags[2:3], self._sym_flags[3:4], self.back if with_forces else None,
                                self._back_idx32 if with_forces else None, force, partial, self._table_ptrs[h], self._table_flag_ptrs[h],
                                self._sym_table[h * P * 16:], self._sym_flags[8 + h * P:], reduced, self.rank, P, self.peer_status,
                                self._counter[1:2])

    # -- the communication steps ---------------------------------------------------------------------
    def halo_exchange(self):
        """Boundary positions (already shifted for the wrap) go straight into the neighbours'
        ghost rows of `local`: one gather, one add on the end slabs, one grouped send/receive."""
        if self.transport == "peer":
            self._peer_halo_exchange()
            return self.local
        if self.P > 1:
            torch.index_select(self.owned, 0, self.send_idx, out=self.send_buf)
            if self.send_shift is not None:
                self.send_buf.add_(self.send_shift)
            self._exchange(self.send_views, self.ghost_views)
        return self.local

    def return_ghost_forces(self, force):
        """force is [ntotal,3]; the rows of the one-cutoff ghosts go back to the ranks that own those atoms
        (into `back`, rows in send-list order)."""
        if self.transport == "peer":
            self._peer_return_ghost_forces(force)
            return
        if self.P > 1:
            nl = len(self.send_lists[0])
            z = force[:0]
            # rows of the ghosts that came from the left go back to the left; what we sent to the left (send list 0,
            # the head of `back`) comes home from the left
            self._exchange([force[self.ghost_slices[0]], force[self.ghost_slices[1]], z, z],
                           [self.back[:nl], self.back[nl:], z, z])

    def add_returned_forces(self, force):
        if self.P > 1:
            force[: self.nlocal].index_add_(0, self.back_idx, self.back)
        return force[: self.nlocal]

    def max_displacement(self):
        """Largest distance an owned atom has moved since set-up (device scalar)."""
        return torch.linalg.norm((self.owned - self.owned_at_setup).double(), dim=1).max() if self.nlocal else torch.zeros((), device=self.device)

    # kept for callers of the first interface: one pass over all owned centres, everything in order
    def evaluate(self, compute):
        """compute(local_coords[ntotal,3], types[ntotal], nlocal, pbc) -> (e[1], f[ntotal,3], v[9])."""
        local = self.halo_exchange()
        e, f, v = compute(local, self.types, self.nlocal, self.pbc)
        f = f.reshape(self.ntotal, 3)
        self.return_ghost_forces(f)
        owned_f = self.add_returned_forces(f)
        ev = torch.cat([e.reshape(1), v.reshape(9)])
        if self.P > 1:
            self.dist.all_reduce(ev)
        return ev[0], owned_f, ev[1:]


class CudaPasses:
    """The per-pass compute on the GPU through the C ABI: neighbour rows for a range of centres
    (ai2b_nblist_build_range_*) and NEP E/F/V added onto the step's accumulators
    (ai2b_nep_efv_accumulate_*). One instance per group of passes that share a set of candidates."""

    def __init__(self, model, cell, rcut, umax, dtype, device, open_extent=None):
        from . import capi
        self.capi = capi
        if model["kind"] != "nep":
            raise ValueError("multi-pass slab evaluation is built for NEP models")
        self.model = capi.to_device({k: v for k, v in model.items() if k != "tables"}, device, dtype)
        self.cell, self.rcut, self.umax, self.ntypes = np.asarray(cell), float(rcut), int(umax), int(model["ntypes"])
        self.dtype, self.device = dtype, device
        self.open_extent = open_extent
        self.builders = {}
        self.slots = {}

    def _slot(self, name, c0, c1, ncand):
        key = (name, c0, c1, ncand)
        s = self.slots.get(key)
        if s is None:
            nc = c1 - c0
            s = dict(out=self.capi.NeighborBuilder.new_outputs(nc, self.umax, self.dtype, self.device),
                     binum=torch.tensor([nc], dtype=torch.int32, device=self.device),
                     bilist=torch.arange(c0, c1, dtype=torch.int32, device=self.device)[None].contiguous(),
                     ws=torch.empty(max(256, self.capi.lib().ai2b_nep_workspace_bytes(1, self.ntypes, int(self.model["n_radial"]),
                                                                                       int(self.model["n_angular"]),
                                                                                       int(self.model["chebyshev_size"]),
                                                                                       1 if self.dtype == torch.float64 else 0)),
                                    dtype=torch.uint8, device=self.device))
            self.slots[key] = s
        return s

    def run_pass(self, name, local, types, c0, c1, ncand, pbc, acc, reuse_bins=False):
        """Adds the contribution of the centres [c0, c1) onto acc = (e[1], f[ntotal,3], v[9]); candidates are the
        atoms [0, ncand). Passes that share `ncand` share a builder, so reuse_bins skips the binning."""
        if c1 <= c0:
            return
        ntotal = local.shape[0]
        s = self._slot(name, c0, c1, ncand)
        b = self.builders.setdefault(ncand, self.capi.NeighborBuilder())
        nn, fn, rcs, status = b.build(self.cell, local[:ncand], self.rcut, self.umax, pbc=pbc, ncentres=c1, cbegin=c0,
                                      reuse_bins=reuse_bins, out=s["out"], open_extent=self.open_extent)
        nc = c1 - c0
        nb = dict(binum=s["binum"], bilist=s["bilist"], bnumneigh=nn[None], bfirstneigh=fn[None], brcs=rcs[None], btypes=types[None],
                  ntypes=self.ntypes, nghost=ntotal - nc)
        e, f, v = acc
        self.capi.nep_efv(self.model, nb, out=(e, f[None], v[None]), accumulate=True, ws=s["ws"])

    def statuses(self):
        return [s["out"][3] for s in self.slots.values()]

    def neighbour_stats(self):
        """(mean neighbours, mean neighbours inside the angular cutoff) over the centres of all passes."""
        tot = ang = cnt = 0.0
        for s in self.slots.values():
            nn, fn, rcs, _ = s["out"]
            tot += float(nn.sum()); cnt += nn.numel()
            inside = (torch.linalg.norm(rcs, dim=-1) <= self.model["rmax_angular"]) & \
                     (torch.arange(rcs.shape[1], device=rcs.device)[None] < nn[:, None])
            ang += float(inside.sum())
        return tot / max(cnt, 1), ang / max(cnt, 1)


class SlabStep:
    """One evaluation of a slab-decomposed system: evaluate() -> (energy, forces of the owned atoms, virial[9]),
    energy and virial already reduced over the ranks. `passes` is a CudaPasses (or, in the CPU tests, any object
    with the same run_pass)."""
    SCHEDULES = ("serial", "overlap", "owner")

    def __init__(self, dom, model=None, umax=None, dtype=None, schedule="serial", passes=None, tail_fraction=0.25, graphs=True):
        if schedule not in self.SCHEDULES:
            raise ValueError(f"schedule must be one of {self.SCHEDULES}")
        if schedule == "owner" and dom.P > 1 and dom.halo_cutoffs < 2:
            raise ValueError("the owner-computes schedule needs a domain built with halo_cutoffs=2")
        if schedule != "owner" and dom.halo_cutoffs != 1:
            raise ValueError("a wide-halo domain only serves the owner-computes schedule")
        self.dom, self.schedule = dom, schedule
        self.cuda = dom.device.type == "cuda"
        self.passes = passes if passes is not None else CudaPasses(model, dom.cell, dom.rcut, umax, dtype, dom.device, dom.open_extent)
        dt = dom.dtype
        # one flat accumulator: [E | virial 9 | 6 unused | forces 3 ntotal], zeroed by one memset per step
        self.flat = torch.zeros(16 + 3 * dom.ntotal, dtype=dt, device=dom.device)
        self.ev = self.flat[:10]
        self.acc = (self.flat[:1], self.flat[16:].view(dom.ntotal, 3), self.flat[1:10])
        self.ev_reduced = torch.zeros(10, dtype=dt, device=dom.device)     # energy / virial summed over the ranks (peer transport)
        # forces-only passes of the owner-computes schedule put their energy / virial here (discarded)
        self.scratch_ev = torch.zeros(16, dtype=dt, device=dom.device)
        # interior centres are split: the tail runs while the ghost forces travel back
        n_int = dom.n_interior
        self.n_head = n_int if (schedule != "overlap" or dom.P == 1) else n_int - int(n_int * tail_fraction)
        self.comm = torch.cuda.Stream(device=dom.device) if (self.cuda and dom.P > 1) else None
        self.use_graphs = bool(graphs) and self.cuda
        self._graphs = {}
        self._prepared = False
        self._segments = self._build_segments()

    # -- compute segments: each a fixed sequence of launches on fixed buffers, replayed from a CUDA graph ---------------
    def _build_segments(self):
        d = self.dom
        n_int, nl = d.n_interior, d.nlocal
        zero = self.flat.zero_
        if d.P == 1:
            return {"all": lambda: (zero(), self._pass("all", 0, nl, nl))}
        if self.schedule == "serial":
            return {"all": lambda: (zero(), self._pass("all", 0, nl, d.ntotal))}
        if self.schedule == "overlap":
            return {"head": lambda: (zero(), self._pass("head", 0, self.n_head, nl)),          # interior centres see owned atoms only
                    "boundary": lambda: self._pass("boundary", n_int, nl, d.ntotal),
                    "tail": lambda: self._pass("tail", self.n_head, n_int, nl, reuse=True)}

        def rest():
            self._pass("boundary", n_int, nl, d.ntotal)
            # ghosts within one cutoff of a face, as centres: only their pair forces on owned atoms are wanted
            self.scratch_ev.zero_()
            self._pass("ghost-centres", nl, nl + d.n_inner_ghost, d.ntotal, acc=(self.scratch_ev[:1], self.acc[1], self.scratch_ev[1:10]),
                       reuse=True)
        return {"head": lambda: (zero(), self._pass("head", 0, n_int, nl)), "rest": rest}

    def _prepare(self):
        """First evaluation: runs the step once without graphs (this sizes every buffer), then records each compute
        segment into a CUDA graph while nothing is in flight. A refused capture leaves that segment eager."""
        self._prepared = True
        self._step()
        torch.cuda.synchronize()
        if self.dom.P > 1:
            self.dom.dist.barrier()
            torch.cuda.synchronize()
        for name, fn in self._segments.items():
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    fn()
                self._graphs[name] = g
            except Exception:
                torch.cuda.synchronize()
        if self.dom.P > 1:
            self.dom.dist.barrier()

    def _seg(self, name):
        g = self._graphs.get(name)
        if g is not None:
            g.replay()
        else:
            self._segments[name]()

    def _pass(self, name, c0, c1, ncand, acc=None, reuse=False):
        d = self.dom
        self.passes.run_pass(name, d.local, d.types, c0, c1, ncand, d.pbc, acc or self.acc, reuse_bins=reuse)

    def evaluate(self):
        if self.use_graphs and not self._prepared:
            self._prepare()
        return self._step()

    def _step(self):
        d = self.dom
        if d.P == 1:
            self._seg("all")
            return self.ev[0], self.acc[1][: d.nlocal], self.ev[1:]
        return getattr(self, "_step_" + self.schedule)()

    def _step_serial(self):
        d = self.dom
        d.halo_exchange()
        self._seg("all")
        if d.transport == "peer":       # force return, accumulation and the reduction of E / virial in one launch
            d.peer_finish(self.acc[1], self.ev, self.ev_reduced)
            return self.ev_reduced[0], self.acc[1][: d.nlocal], self.ev_reduced[1:]
        d.return_ghost_forces(self.acc[1])
        owned_f = d.add_returned_forces(self.acc[1])
        d.dist.all_reduce(self.ev)
        return self.ev[0], owned_f, self.ev[1:]

    def _on_comm(self, fn):
        """Runs fn on the communication stream after everything issued so far on the main stream; returns an
        event the main stream can wait on. Without a second stream (CPU ranks) fn runs in line."""
        if self.comm is None:
            fn()
            return None
        self.comm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm):
            fn()
            ev = torch.cuda.Event()
            ev.record(self.comm)
        return ev

    @staticmethod
    def _wait(ev):
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _step_overlap(self):
        d = self.dom
        halo = self._on_comm(d.halo_exchange)
        self._seg("head")                               # runs while the halo is in flight
        self._wait(halo)
        self._seg("boundary")
        back = self._on_comm(lambda: d.return_ghost_forces(self.acc[1]))     # ghost rows are final: interior passes never touch them
        self._seg("tail")                               # runs while the ghost forces travel back
        self._wait(back)
        owned_f = d.add_returned_forces(self.acc[1])
        d.dist.all_reduce(self.ev)
        return self.ev[0], owned_f, self.ev[1:]

    def _step_owner(self):
        d = self.dom
        halo = self._on_comm(d.halo_exchange)
        self._seg("head")
        self._wait(halo)
        self._seg("rest")
        if d.transport == "peer":
            d.peer_finish(self.acc[1], self.ev, self.ev_reduced, with_forces=False)
            return self.ev_reduced[0], self.acc[1][: d.nlocal], self.ev_reduced[1:]
        d.dist.all_reduce(self.ev)
        return self.ev[0], self.acc[1][: d.nlocal], self.ev[1:]

    # -- bookkeeping for the benchmark ---------------------------------------------------------------------
    def check_status(self):
        """Raises if a neighbour row overflowed umax or an owned atom has moved more than half the skin since set-up."""
        for st in self.passes.statuses():
            s = st.cpu().numpy()
            if s[1]:
                raise RuntimeError(f"umax too small (largest neighbour count {int(s[0])})")
        if self.dom.transport == "peer" and int(self.dom.peer_status[0]):
            from .capi import Ai2bError, AI2B_ERR_TIMEOUT
            raise Ai2bError(f"ai2pot_b200 error {AI2B_ERR_TIMEOUT}: a neighbour's halo or ghost-force rows did not arrive within the wait limit")
        moved = float(self.dom.max_displacement())
        if moved > 0.5 * self.dom.skin + 1e-6:
            raise RuntimeError(f"an atom moved {moved:.3g} since the domain was set up (skin {self.dom.skin}): build a new SlabDomain")

    def neighbour_stats(self):
        return self.passes.neighbour_stats()

    def halo_bytes(self):
        d = self.dom
        return int(d.send_buf.numel() * d.send_buf.element_size()) if d.P > 1 else 0

    def return_bytes(self):
        d = self.dom
        return int(d.back.numel() * d.back.element_size()) if (d.P > 1 and self.schedule != "owner") else 0

    def launches_per_step(self):
        """Kernels of this library per step: a pass = neighbour build (set-up, count, scan, fill, rows; rows only when
        the bins are reused) + one NEP kernel."""
        if self.dom.P == 1 or self.schedule == "serial":
            return 6
        return 6 + 6 + 2

    def parts_ms(self, k, flush, timed):
        """Device times of the parts of a step run one at a time (not overlapped), for the record."""
        d = self.dom
        out = {}
        if d.P > 1:
            out["halo_exchange"] = 1e3 * timed(d.halo_exchange, k, 2, flush) / k
            if self.schedule != "owner":
                out["ghost_force_return"] = 1e3 * timed(lambda: d.return_ghost_forces(self.acc[1]), k, 2, flush) / k
            tmp = torch.zeros(10, dtype=d.dtype, device=d.device)
            out["allreduce_e_virial"] = 1e3 * timed(lambda: d.dist.all_reduce(tmp), k, 2, flush) / k
        total = 0.0
        for n in self._segments:
            t = 1e3 * timed(lambda: self._seg(n), k, 2, flush) / k
            out["pass_" + n] = t
            total += t
        out["nblist+efv"] = total
        return out


class LocalCompute:
    """One pass over all owned centres on the GPU through the C ABI (the compute of SlabDomain.evaluate):
    ghost-aware neighbour list, then NEP or MTP E/F/V."""

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
