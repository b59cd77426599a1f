"""Host-side driver of the evaluation path: positions -> neighbour list -> E/F/V on one GPU.
Everything on the device goes through the C ABI."""
import numpy as np
import torch

from . import capi


class Evaluator:
    """One structure, one model, one GPU: compute(coords) -> (etot[1], force[1,N,3], virial[1,9]).
    Mirrors what the reference's calculators do per call (neighbour list, then predict_efv:
    ai2pot/models/potential_utils.py:217-268), with every step on the device."""

    def __init__(self, model, cell, types, rcut, umax, dtype):
        self.kind = model["kind"]
        self.dtype = dtype
        self.cell = np.asarray(cell)
        self.rcut, self.umax = float(rcut), int(umax)
        n = len(types)
        self.n = n
        dev = torch.device("cuda", torch.cuda.current_device())
        self.model = capi.to_device({k: v for k, v in model.items() if k != "tables"}, dev, dtype)
        self.prog = capi.MtpProgram(model["tables"]) if self.kind == "mtp" else None
        self.builder = capi.NeighborBuilder()
        self.nb_static = dict(binum=torch.tensor([n], dtype=torch.int32, device=dev),
                              bilist=torch.arange(n, dtype=torch.int32, device=dev)[None].contiguous(),
                              btypes=torch.from_numpy(np.ascontiguousarray(types, np.int32)).to(dev)[None].contiguous(),
                              ntypes=int(model["ntypes"]), nghost=0)
        # E, virial and forces in one piece, [E | virial (9) | pad | forces (3 n)], so that a host reads them with one copy
        self.outbuf = torch.empty(16 + 3 * n, dtype=dtype, device=dev)
        self.out = (self.outbuf[0:1], self.outbuf[16:].view(1, n, 3), self.outbuf[1:10].view(1, 9))
        self.status = None
        self.graph = self.graph_io = None

    def build_list(self, coords):
        nn, fn, rcs, status = self.builder.build(self.cell, coords, self.rcut, self.umax)
        self.status = status
        return dict(self.nb_static, bnumneigh=nn[None], bfirstneigh=fn[None], brcs=rcs[None])

    def evaluate(self, nb):
        if self.kind == "mtp":
            return capi.mtp_efv(self.prog, self.model, nb, out=self.out)
        return capi.nep_efv(self.model, nb, out=self.out)

    def compute(self, coords):
        return self.evaluate(self.build_list(coords))

    def capture(self, coords):
        """Records one compute(coords) (neighbour build + E/F/V, every launch stream-ordered on buffers this
        object owns) into a CUDA graph; replay() then re-runs it on whatever `coords` holds at that time.
        Returns False (and leaves the eager path in place) if the capture is refused."""
        self.graph = None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.compute(coords)                      # sizes every buffer before the capture
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.graph_out = self.compute(coords)
            self.graph = g
        except Exception:
            self.graph = None
            torch.cuda.synchronize()
        return self.graph is not None

    def replay(self):
        self.graph.replay()
        return self.graph_out

    def capture_io(self, coords, host_coords, host_out):
        """One CUDA graph for a whole call as a host sees it: pinned host positions -> device, neighbour build, E/F/V,
        results -> pinned host buffer `host_out` (laid out like `outbuf`: E, virial 1..9, forces from element 16).
        replay_io() then costs one graph launch. Returns False if the capture is refused."""
        self.graph_io = None
        try:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                coords.copy_(host_coords, non_blocking=True)
                self.compute(coords)
                host_out.copy_(self.outbuf, non_blocking=True)
            self.graph_io = g
        except Exception:
            self.graph_io = None
            torch.cuda.synchronize()
        return self.graph_io is not None

    def replay_io(self):
        self.graph_io.replay()

    # kernels of this library launched by one compute() on a fully periodic cell (memsets not counted):
    # neighbour build = set-up, count, scan, fill, build; MTP = forward, contraction, force (plus a set-up launch when the
    # radial coefficient rows have to be padded to eight entries); NEP = zeroing of the outputs + one kernel
    def launches_per_step(self):
        if self.kind == "mtp":
            return 5 + 3 + (0 if int(self.model["chebyshev_size"]) == 8 else 1)
        return 5 + 2
