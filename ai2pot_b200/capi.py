"""ctypes binding of the C ABI declared in include/ai2pot_b200.h.

PyTorch is used only as the owner of device memory and streams: every function here takes torch
CUDA tensors, passes their raw pointers to libai2pot_b200.so and returns torch tensors. There is
no CPU implementation behind these calls: a missing library or a non-CUDA tensor raises.
"""
import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libai2pot_b200.so")
_lib = None


class Ai2bError(RuntimeError):
    pass


def lib():
    """The loaded CUDA library. Raises if it has not been built (python -m ai2pot_b200._build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Ai2bError(f"{LIB_PATH} is missing: build it with `python -m ai2pot_b200._build` "
                            "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.ai2b_last_error_string.restype = C.c_char_p
        _lib.ai2b_mtp_workspace_bytes.restype = C.c_size_t
        _lib.ai2b_nblist_workspace_bytes.restype = C.c_size_t
        _lib.ai2b_nep_workspace_bytes.restype = C.c_size_t
        _lib.ai2b_mtp_loss_workspace_bytes.restype = C.c_size_t
    return _lib


def _check(rc):
    if rc != 0:
        raise Ai2bError(f"ai2pot_b200 error {rc}: {lib().ai2b_last_error_string().decode()}")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise Ai2bError("expected a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise Ai2bError("expected a contiguous tensor")
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _suf(dtype):
    if dtype == torch.float64:
        return "f64", C.c_double
    if dtype == torch.float32:
        return "f32", C.c_float
    raise Ai2bError(f"unsupported float dtype {dtype}")


def to_device(d, device="cuda", float_dtype=None):
    """Copy the numpy arrays of a dict (model parameters or neighbour tensors) to the device."""
    out = {}
    for k, v in d.items():
        if isinstance(v, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(v))
            if float_dtype is not None and t.is_floating_point():
                t = t.to(float_dtype)
            out[k] = t.to(device)
        else:
            out[k] = v
    return out


class MtpProgram:
    """Compiled alpha tables (ai2b_mtp_program). `tables` holds host int32 arrays."""

    def __init__(self, tables):
        self.tables = tables
        b = np.ascontiguousarray(tables["alpha_index_basic"], np.int32)
        t = np.ascontiguousarray(tables["alpha_index_times"], np.int32)
        m = np.ascontiguousarray(tables["alpha_moment_mapping"], np.int32)
        self.ns = len(m)
        self.nmus = int(tables["nmus"])
        self.handle = C.c_void_p()
        _check(lib().ai2b_mtp_program_create(
            C.c_int(int(tables["alpha_moments_count"])), C.c_int(len(b)), b.ctypes.data_as(C.c_void_p),
            C.c_int(len(t)), t.ctypes.data_as(C.c_void_p), C.c_int(len(m)), m.ctypes.data_as(C.c_void_p),
            C.c_int(self.nmus), C.byref(self.handle)))
        self._ws = None

    def workspace(self, B, npad, ntypes, device):
        need = lib().ai2b_mtp_workspace_bytes(self.handle, C.c_int(B), C.c_int(npad), C.c_int(ntypes))
        if self._ws is None or self._ws.numel() < need or self._ws.device != device:
            self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
        return self._ws

    def __del__(self):
        try:
            if self.handle:
                lib().ai2b_mtp_program_destroy(self.handle)
        except Exception:
            pass


def parse_almtp(path):
    """Parse an MTP template file with the library's own parser -> tables dict."""
    counts = np.zeros(5, np.int32)
    _check(lib().ai2b_mtp_parse_almtp(path.encode(), counts.ctypes.data_as(C.c_void_p), None, None, None))
    b = np.zeros((counts[1], 4), np.int32); t = np.zeros((counts[2], 4), np.int32); m = np.zeros(counts[3], np.int32)
    _check(lib().ai2b_mtp_parse_almtp(path.encode(), counts.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p),
                                      t.ctypes.data_as(C.c_void_p), m.ctypes.data_as(C.c_void_p)))
    return dict(alpha_moments_count=int(counts[0]), nmus=int(counts[4]), alpha_index_basic=b,
                alpha_index_times=t, alpha_moment_mapping=m)


def _nb_args(nb):
    B, npad = nb["bilist"].shape
    umax = nb["bfirstneigh"].shape[2]
    return B, npad, umax, (C.c_int(B), C.c_int(npad), _ptr(nb["binum"]), _ptr(nb["bilist"]), _ptr(nb["bnumneigh"]),
                           _ptr(nb["bfirstneigh"]), _ptr(nb["brcs"]), _ptr(nb["btypes"]), C.c_int(int(nb["ntypes"])),
                           C.c_int(umax), C.c_int(int(nb.get("nghost", 0))))


def mtp_efv(prog, model, nb, virial=True, out=None):
    """Energy, forces (and virial) of a batch. `model` / `nb` hold device tensors (see to_device)."""
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, nbargs = _nb_args(nb)
    ng = int(nb.get("nghost", 0))
    if out is None:
        e = torch.empty(B, dtype=rcs.dtype, device=rcs.device)
        f = torch.empty(B, npad + ng, 3, dtype=rcs.dtype, device=rcs.device)
        v = torch.empty(B, 9, dtype=rcs.dtype, device=rcs.device) if virial else None
    else:
        e, f, v = out
    ws = prog.workspace(B, npad, int(nb["ntypes"]), rcs.device)
    _check(getattr(lib(), "ai2b_mtp_efv_" + suf)(
        prog.handle, _ptr(e), _ptr(f), _ptr(v), C.c_int(int(model["chebyshev_size"])), cf(model["scaling"]),
        _ptr(model["coeffs"]), _ptr(model["linear_coeffs"]), _ptr(model["type_bias"]), *nbargs,
        cf(model["rmax"]), cf(model["rmin"]), _ptr(model["q_scaler"]), _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return (e, f, v) if virial else (e, f)


def mtp_descriptors(prog, model, nb):
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, nbargs = _nb_args(nb)
    d = torch.empty(B, npad, prog.ns, dtype=rcs.dtype, device=rcs.device)
    ws = prog.workspace(B, npad, int(nb["ntypes"]), rcs.device)
    _check(getattr(lib(), "ai2b_mtp_descriptors_" + suf)(
        prog.handle, _ptr(d), C.c_int(int(model["chebyshev_size"])), cf(model["scaling"]), _ptr(model["coeffs"]),
        *nbargs, cf(model["rmax"]), cf(model["rmin"]), _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return d


class NeighborBuilder:
    """Device neighbour-list builder for one structure (ai2b_nblist_build_*). Keeps its workspace
    and output tensors between calls, so repeated builds of same-sized systems allocate nothing."""

    def __init__(self):
        self._ws = None
        self._out = None

    @staticmethod
    def new_outputs(nc, umax, dtype, dev):
        return (torch.empty(nc, dtype=torch.int32, device=dev), torch.empty(nc, umax, dtype=torch.int32, device=dev),
                torch.empty(nc, umax, 3, dtype=dtype, device=dev), torch.zeros(2, dtype=torch.int32, device=dev))

    def build(self, cell, coords, rcut, umax, is_cart=True, pbc=(True, True, True), ncentres=None, cbegin=0, reuse_bins=False,
              out=None, open_extent=None):
        """cell: host array [3,3]; coords: CUDA tensor [N,3] (float32/float64). With `ncentres`
        rows are built for the atoms [cbegin, ncentres) only (the rest are candidates only, e.g. ghosts);
        reuse_bins: this builder's workspace still holds the binning of the same atoms (see
        ai2b_nblist_build_range_*).
        open_extent: (lo, hi) fractional bounds of the atoms along a non-periodic first axis, if the caller knows them.
        out: (numneigh, firstneigh, rcs, status) tensors of the caller to write into (several passes that share
        one builder keep their own outputs).
        Returns (numneigh[Nc], firstneigh[Nc,umax], rcs[Nc,umax,3], status[2]) device tensors, Nc = ncentres - cbegin."""
        if not coords.is_cuda:
            raise Ai2bError("coords must be a CUDA tensor")
        suf, _ = _suf(coords.dtype)
        n = coords.shape[0]
        npdt = np.float64 if suf == "f64" else np.float32
        hcell = np.ascontiguousarray(np.asarray(cell, dtype=npdt).reshape(9))
        hpbc = np.ascontiguousarray([1 if p else 0 for p in pbc], np.int32)
        need = lib().ai2b_nblist_workspace_bytes(C.c_int(n), C.c_int(1 if suf == "f64" else 0))
        dev = coords.device
        if self._ws is None or self._ws.numel() < need or self._ws.device != dev:
            self._ws = torch.empty(need, dtype=torch.uint8, device=dev)
        cend = n if ncentres is None else int(ncentres)
        nc = cend - int(cbegin)
        if out is not None:
            nn, fn, rcs, status = out
        else:
            key = (nc, umax, coords.dtype, dev)
            if self._out is None or self._out[0] != key:
                self._out = (key,) + self.new_outputs(nc, umax, coords.dtype, dev)
            _, nn, fn, rcs, status = self._out
        coords = coords.contiguous()
        ext = None
        if open_extent is not None and not all(pbc):
            hext = np.ascontiguousarray([open_extent[0], 0.0, 0.0, open_extent[1], 1.0, 1.0], np.float64)
            if pbc[0] or not (pbc[1] and pbc[2]):
                raise Ai2bError("open_extent is taken for a cell that is open along its first axis only")
            ext = hext.ctypes.data_as(C.c_void_p)
        _check(getattr(lib(), "ai2b_nblist_build_range_" + suf)(
            C.c_int(n), C.c_int(int(cbegin)), C.c_int(cend), hcell.ctypes.data_as(C.c_void_p), _ptr(coords), C.c_int(1 if is_cart else 0),
            C.c_double(rcut), hpbc.ctypes.data_as(C.c_void_p), ext, C.c_int(umax), C.c_int(1 if reuse_bins else 0), _ptr(nn), _ptr(fn),
            _ptr(rcs), _ptr(status), _ptr(self._ws), C.c_size_t(self._ws.numel()), _stream()))
        return nn, fn, rcs, status


def nblist_build_batch(cells, binum, coords, rcut, umax, is_cart=True, pbc=(True, True, True)):
    """Neighbour tensors of a padded batch in one launch (ai2b_nblist_build_batch_*).
    cells: host array [B,3,3]; binum: CUDA int32 [B]; coords: CUDA [B,Np,3] (float32/float64).
    Returns a dict with binum, bilist, bnumneigh, bfirstneigh, brcs, status (device tensors)."""
    if not coords.is_cuda:
        raise Ai2bError("coords must be a CUDA tensor")
    suf, _ = _suf(coords.dtype)
    B, npad = int(coords.shape[0]), int(coords.shape[1])
    dev = coords.device
    npdt = np.float64 if suf == "f64" else np.float32
    dcells = torch.from_numpy(np.ascontiguousarray(np.asarray(cells, dtype=npdt).reshape(B, 9))).to(dev)
    hpbc = np.ascontiguousarray([1 if p else 0 for p in pbc], np.int32)
    binum = binum.to(torch.int32).contiguous()
    out = dict(binum=binum, bilist=torch.empty(B, npad, dtype=torch.int32, device=dev),
               bnumneigh=torch.empty(B, npad, dtype=torch.int32, device=dev),
               bfirstneigh=torch.empty(B, npad, umax, dtype=torch.int32, device=dev),
               brcs=torch.empty(B, npad, umax, 3, dtype=coords.dtype, device=dev),
               status=torch.zeros(2, dtype=torch.int32, device=dev))
    _check(getattr(lib(), "ai2b_nblist_build_batch_" + suf)(
        C.c_int(B), C.c_int(npad), _ptr(binum), _ptr(dcells), _ptr(coords.contiguous()), C.c_int(1 if is_cart else 0), C.c_double(rcut),
        hpbc.ctypes.data_as(C.c_void_p), C.c_int(umax), _ptr(out["bilist"]), _ptr(out["bnumneigh"]), _ptr(out["bfirstneigh"]),
        _ptr(out["brcs"]), _ptr(out["status"]), _stream()))
    return out


def sort_rows_by_distance(numneigh, firstneigh, rcs):
    """In-place distance ordering of every row (ai2b_nblist_sort_rows_*)."""
    suf, _ = _suf(rcs.dtype)
    n, umax = firstneigh.shape
    _check(getattr(lib(), "ai2b_nblist_sort_rows_" + suf)(C.c_int(n), C.c_int(umax), _ptr(numneigh), _ptr(firstneigh),
                                                          _ptr(rcs), _stream()))
    return numneigh, firstneigh, rcs


_nep_ws = {}


def _nep_workspace(model, B, dtype, device):
    need = lib().ai2b_nep_workspace_bytes(C.c_int(B), C.c_int(int(model["ntypes"])), C.c_int(int(model["n_radial"])),
                                          C.c_int(int(model["n_angular"])), C.c_int(int(model["chebyshev_size"])),
                                          C.c_int(1 if dtype == torch.float64 else 0))
    ws = _nep_ws.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _nep_ws[device] = ws
    return ws


def nep_efv(model, nb, virial=True, out=None, accumulate=False, ws=None):
    """NEP energy, forces (and virial) of a batch; `model` / `nb` hold device tensors. accumulate: add onto
    `out` (ai2b_nep_efv_accumulate_*) instead of overwriting it. ws: a workspace tensor of the caller (calls
    that may run concurrently on different streams must not share one)."""
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, nbargs = _nb_args(nb)
    ng = int(nb.get("nghost", 0))
    if out is None:
        e = torch.empty(B, dtype=rcs.dtype, device=rcs.device)
        f = torch.empty(B, npad + ng, 3, dtype=rcs.dtype, device=rcs.device)
        v = torch.empty(B, 9, dtype=rcs.dtype, device=rcs.device) if virial else None
    else:
        e, f, v = out
    if ws is None:
        ws = _nep_workspace(model, B, rcs.dtype, rcs.device)
    _check(getattr(lib(), ("ai2b_nep_efv_accumulate_" if accumulate else "ai2b_nep_efv_") + suf)(
        _ptr(e), _ptr(f), _ptr(v), C.c_int(int(model["chebyshev_size"])), C.c_int(int(model["n_radial"])),
        C.c_int(int(model["n_angular"])), C.c_int(int(model["l_max"])), C.c_int(int(model["num_neurons"])),
        _ptr(model["coeffs"]), _ptr(model["w0"]), _ptr(model["b0"]), _ptr(model["w1"]), _ptr(model["type_bias"]),
        *nbargs, cf(model["rmax_radial"]), cf(model["rmax_angular"]), _ptr(model["q_scaler"]), _ptr(ws),
        C.c_size_t(ws.numel()), _stream()))
    return (e, f, v) if virial else (e, f)


def nep_loss_backward(model, nb, weights, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
    """Per-structure gradients of the NEP loss: (dcoeffs [B,ncoef], dw0 [B,nt*nneu*nd], db0, dw1 [B,nt*nneu], dbias [B,nt])."""
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, _ = _nb_args(nb)
    nt, nneu = int(nb["ntypes"]), int(model["num_neurons"])
    nd = int(model["n_radial"]) + int(model["n_angular"]) * int(model["l_max"])
    mk = lambda n: torch.empty(B, n, dtype=rcs.dtype, device=rcs.device)
    dco, dw0, db0, dw1, dbi = mk(model["coeffs"].numel()), mk(nt * nneu * nd), mk(nt * nneu), mk(nt * nneu), mk(nt)
    _check(getattr(lib(), "ai2b_nep_loss_backward_" + suf)(
        _ptr(dco), _ptr(dw0), _ptr(db0), _ptr(dw1), _ptr(dbi), cf(weights[0]), cf(weights[1]), cf(weights[2] if len(weights) > 2 else 0.0),
        _ptr(e_ml), _ptr(e_dft), _ptr(f_ml), _ptr(f_dft), _ptr(v_ml), _ptr(v_dft), C.c_int(int(model["chebyshev_size"])),
        C.c_int(int(model["n_radial"])), C.c_int(int(model["n_angular"])), C.c_int(int(model["l_max"])), C.c_int(nneu),
        _ptr(model["coeffs"]), _ptr(model["w0"]), _ptr(model["b0"]), _ptr(model["w1"]), C.c_int(B), C.c_int(npad), _ptr(nb["binum"]),
        _ptr(nb["bilist"]), _ptr(nb["bnumneigh"]), _ptr(nb["bfirstneigh"]), _ptr(rcs), _ptr(nb["btypes"]), C.c_int(nt), C.c_int(umax),
        C.c_int(int(nb.get("nghost", 0))), cf(model["rmax_radial"]), cf(model["rmax_angular"]), _ptr(model["q_scaler"]), _stream()))
    return dco, dw0, db0, dw1, dbi


def weighted_sum_rows(parts, w=None, out=None):
    """out = concatenation over k of (w @ parts[k].reshape(B, -1)); w None: sums over the first axis.
    One launch for up to 8 per-structure gradient tensors (ai2b_weighted_sum_rows)."""
    parts = [p_.contiguous() for p_ in parts]
    B = parts[0].shape[0]
    dt, dev = parts[0].dtype, parts[0].device
    suf, cf = _suf(dt)
    ns = [p_.numel() // B if B else 0 for p_ in parts]
    if out is None:
        out = torch.empty(sum(ns), dtype=dt, device=dev)
    assert out.numel() == sum(ns) and out.dtype == dt and out.is_contiguous()
    if sum(ns) == 0:
        return out
    ptrs = (C.c_void_p * len(parts))(*[p_.data_ptr() for p_ in parts])
    n_arr = (C.c_int * len(parts))(*ns)
    _check(getattr(lib(), "ai2b_weighted_sum_rows_" + suf)(C.c_int(len(parts)), ptrs, n_arr, C.c_int(B),
                                                          _ptr(w.contiguous()) if w is not None else None, _ptr(out), _stream()))
    return out


def zbl_efv(nb, type_map, rmax, rmin, cks, dks, e, f, v=None):
    """Adds the ZBL pair correction onto e[B], f[B,Np+nghost,3] and (if given) v[B,9] in place.
    type_map: int32 atomic numbers [ntypes]; cks, dks: [ntypes*ntypes*4] (device tensors)."""
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad = nb["bilist"].shape
    umax = nb["bfirstneigh"].shape[2]
    _check(getattr(lib(), "ai2b_zbl_efv_" + suf)(
        _ptr(e), _ptr(f), _ptr(v), C.c_int(B), C.c_int(npad), _ptr(nb["binum"]), _ptr(nb["bilist"]), _ptr(nb["bnumneigh"]),
        _ptr(nb["bfirstneigh"]), _ptr(rcs), _ptr(nb["btypes"]), C.c_int(int(nb["ntypes"])), _ptr(type_map), C.c_int(umax),
        C.c_int(int(nb.get("nghost", 0))), cf(rmax), cf(rmin), _ptr(cks), _ptr(dks), _stream()))
    return e, f, v


def nep_descriptors(model, nb):
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, nbargs = _nb_args(nb)
    nd = int(model["n_radial"]) + int(model["n_angular"]) * int(model["l_max"])
    d = torch.empty(B, npad, nd, dtype=rcs.dtype, device=rcs.device)
    ws = _nep_workspace(model, B, rcs.dtype, rcs.device)
    _check(getattr(lib(), "ai2b_nep_descriptors_" + suf)(
        _ptr(d), C.c_int(int(model["chebyshev_size"])), C.c_int(int(model["n_radial"])), C.c_int(int(model["n_angular"])),
        C.c_int(int(model["l_max"])), _ptr(model["coeffs"]), *nbargs, cf(model["rmax_radial"]), cf(model["rmax_angular"]),
        _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return d


def mtp_loss(nb, weights, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
    """Per-structure loss [B] and rmse[3] = (energy, force, virial)."""
    suf, cf = _suf(e_ml.dtype)
    B, npad = nb["bilist"].shape
    loss = torch.empty(B, dtype=e_ml.dtype, device=e_ml.device)
    rmse = torch.empty(3, dtype=e_ml.dtype, device=e_ml.device)
    ws = torch.empty(256, dtype=torch.uint8, device=e_ml.device)
    _check(getattr(lib(), "ai2b_mtp_loss_" + suf)(
        _ptr(loss), _ptr(rmse), C.c_int(B), C.c_int(npad), C.c_int(int(nb.get("nghost", 0))), _ptr(nb["binum"]), _ptr(nb["bilist"]),
        cf(weights[0]), cf(weights[1]), cf(weights[2]), _ptr(e_ml), _ptr(e_dft), _ptr(f_ml), _ptr(f_dft), _ptr(v_ml), _ptr(v_dft),
        _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return loss, rmse


def nep_loss(nb, weights, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
    """As mtp_loss, with the NEP ops' per-atom energy RMSE in rmse[0]."""
    suf, cf = _suf(e_ml.dtype)
    B, npad = nb["bilist"].shape
    loss = torch.empty(B, dtype=e_ml.dtype, device=e_ml.device)
    rmse = torch.empty(3, dtype=e_ml.dtype, device=e_ml.device)
    ws = torch.empty(256, dtype=torch.uint8, device=e_ml.device)
    _check(getattr(lib(), "ai2b_nep_loss_" + suf)(
        _ptr(loss), _ptr(rmse), C.c_int(B), C.c_int(npad), C.c_int(int(nb.get("nghost", 0))), _ptr(nb["binum"]), _ptr(nb["bilist"]),
        cf(weights[0]), cf(weights[1]), cf(weights[2]), _ptr(e_ml), _ptr(e_dft), _ptr(f_ml), _ptr(f_dft), _ptr(v_ml), _ptr(v_dft),
        _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return loss, rmse


def mtp_loss_backward(prog, model, nb, weights, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
    """Per-structure gradients (dcoeffs [B,ncoef], dlinear [B,ns], dbias [B,ntypes])."""
    rcs = nb["brcs"]
    suf, cf = _suf(rcs.dtype)
    B, npad, umax, nbargs = _nb_args(nb)
    ntypes = int(nb["ntypes"])
    dco = torch.empty(B, model["coeffs"].numel(), dtype=rcs.dtype, device=rcs.device)
    dli = torch.empty(B, prog.ns, dtype=rcs.dtype, device=rcs.device)
    dbi = torch.empty(B, ntypes, dtype=rcs.dtype, device=rcs.device)
    need = lib().ai2b_mtp_loss_workspace_bytes(prog.handle, C.c_int(B), C.c_int(npad), C.c_int(ntypes))
    ws = torch.empty(need, dtype=torch.uint8, device=rcs.device)
    _check(getattr(lib(), "ai2b_mtp_loss_backward_" + suf)(
        prog.handle, _ptr(dco), _ptr(dli), _ptr(dbi), cf(weights[0]), cf(weights[1]), cf(weights[2]), _ptr(e_ml), _ptr(e_dft),
        _ptr(f_ml), _ptr(f_dft), _ptr(v_ml), _ptr(v_dft), C.c_int(int(model["chebyshev_size"])), cf(model["scaling"]),
        _ptr(model["coeffs"]), _ptr(model["linear_coeffs"]), _ptr(model["type_bias"]), *nbargs, cf(model["rmax"]), cf(model["rmin"]),
        _ptr(model["q_scaler"]), _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return dco, dli, dbi


AI2B_ERR_TIMEOUT = -6


def peer_push_rows(src, src_index, dst_index, nrows, shift3, peer_dst, peer_flag, flag_value, counter):
    """ai2b_peer_push_rows_*: peer_dst[dst_index[k]] = src[src_index[k]] + shift3 for k < nrows, then the flag
    (an int32 element of the neighbour's flag tensor) is set to flag_value. All tensors are CUDA tensors; peer_dst
    and peer_flag alias the neighbour's memory."""
    suf, _ = _suf(src.dtype)
    npdt = np.float64 if suf == "f64" else np.float32
    sh = None
    if shift3 is not None:
        hs = np.ascontiguousarray(shift3, npdt)
        sh = hs.ctypes.data_as(C.c_void_p)
    _check(getattr(lib(), "ai2b_peer_push_rows_" + suf)(
        _ptr(src), _ptr(src_index), _ptr(dst_index), C.c_int(int(nrows)), sh, C.c_void_p(peer_dst.data_ptr()),
        C.c_void_p(peer_flag.data_ptr()), C.c_int(int(flag_value)), _ptr(counter), _stream()))


def peer_exchange(left, right, flag_value, my_flag_l, my_flag_r, status, counter, max_polls=20_000_000):
    """ai2b_peer_exchange_*: both pushes of an exchange and the wait for the neighbours' pushes in one launch.
    left / right: dict(src, src_idx, dst_idx, n, shift, dst, flag) as for peer_push_rows."""
    suf, _ = _suf(left["src"].dtype)
    npdt = np.float64 if suf == "f64" else np.float32
    keep = []

    def side(p):
        sh = None
        if p.get("shift") is not None:
            hs = np.ascontiguousarray(p["shift"], npdt)
            keep.append(hs)
            sh = hs.ctypes.data_as(C.c_void_p)
        return (_ptr(p["src"]), _ptr(p.get("src_idx")), _ptr(p.get("dst_idx")), C.c_int(int(p["n"])), sh,
                C.c_void_p(p["dst"].data_ptr()), C.c_void_p(p["flag"].data_ptr()))
    _check(getattr(lib(), "ai2b_peer_exchange_" + suf)(*side(left), *side(right), C.c_int(int(flag_value)), _ptr(my_flag_l), _ptr(my_flag_r),
                                                       C.c_longlong(int(max_polls)), _ptr(status), _ptr(counter), _stream()))


def peer_return_reduce(left, right, flag_value, my_flag_l, my_flag_r, back, back_index, force, partial, peer_tables, peer_table_flags,
                       my_table, my_table_flags, reduced, rank, nranks, status, counter, max_polls=20_000_000):
    """ai2b_peer_return_reduce_*: ghost-force rows to both neighbours, partial sums to every rank, then the received
    rows added onto `force` and the partials of all ranks summed into `reduced`, in one launch. left / right:
    dict(src, n, dst, flag) or None; peer_tables / peer_table_flags: int64 CUDA tensors of device addresses."""
    suf, _ = _suf(force.dtype)

    def side(p):
        if p is None or p["n"] == 0:
            return (None, C.c_int(0), None, None if p is None else C.c_void_p(p["flag"].data_ptr()))
        return (_ptr(p["src"]), C.c_int(int(p["n"])), C.c_void_p(p["dst"].data_ptr()), C.c_void_p(p["flag"].data_ptr()))
    nback = 0 if back_index is None else int(back_index.numel())
    nvalues = int(partial.numel())
    _check(getattr(lib(), "ai2b_peer_return_reduce_" + suf)(
        *side(left), *side(right), C.c_int(int(flag_value)), _ptr(my_flag_l), _ptr(my_flag_r), _ptr(back) if nback else None,
        _ptr(back_index) if nback else None, C.c_int(nback), _ptr(force), _ptr(partial), _ptr(peer_tables), _ptr(peer_table_flags),
        _ptr(my_table), _ptr(my_table_flags), _ptr(reduced), C.c_int(int(rank)), C.c_int(int(nranks)), C.c_int(nvalues),
        C.c_longlong(int(max_polls)), _ptr(status), _ptr(counter), _stream()))


def peer_wait(flag, value, status, max_polls=5_000_000):
    """ai2b_peer_wait: the current stream waits until flag[0] >= value, for at most max_polls polls of 200 ns;
    a wait that gives up stores 1 to status[0]."""
    _check(lib().ai2b_peer_wait(_ptr(flag), C.c_int(int(value)), C.c_longlong(int(max_polls)), _ptr(status), _stream()))


class MdSession:
    """ctypes wrapper of ai2b_md_session_*: the device-resident input path of an MD host
    (positions + model types in, forces on local and ghost atoms + energy + six virial components out).
    `model` holds numpy arrays (see synth.nep_model / synth.mtp_model); for MTP pass the MtpProgram too."""

    def __init__(self, model, umax, prog=None):
        self.h = C.c_void_p()
        f32 = lambda a: np.ascontiguousarray(np.asarray(a).ravel(), np.float32)
        hp = lambda a: a.ctypes.data_as(C.c_void_p)
        self.kind = model["kind"]
        if self.kind == "nep":
            a = [f32(model[k]) for k in ("coeffs", "w0", "b0", "w1", "type_bias", "q_scaler")]
            _check(lib().ai2b_md_session_create_nep(
                C.byref(self.h), C.c_int(int(model["chebyshev_size"])), C.c_int(int(model["n_radial"])), C.c_int(int(model["n_angular"])),
                C.c_int(int(model["l_max"])), C.c_int(int(model["num_neurons"])), C.c_int(int(model["ntypes"])), *[hp(x) for x in a],
                C.c_float(model["rmax_radial"]), C.c_float(model["rmax_angular"]), C.c_int(int(umax))))
        else:
            self.prog = prog
            a = [f32(model[k]) for k in ("coeffs", "linear_coeffs", "type_bias", "q_scaler")]
            _check(lib().ai2b_md_session_create_mtp(
                C.byref(self.h), prog.handle, C.c_int(int(model["chebyshev_size"])), C.c_float(model["scaling"]),
                C.c_int(int(model["ntypes"])), C.c_int(int(prog.nmus)), C.c_int(int(prog.ns)), *[hp(x) for x in a],
                C.c_float(model["rmax"]), C.c_float(model["rmin"]), C.c_int(int(umax))))

    def compute(self, nlocal, nghost, x, model_type, want_virial=True):
        x = np.ascontiguousarray(x, np.float64)
        t = np.ascontiguousarray(model_type, np.int32)
        f = np.zeros((nlocal + nghost, 3), np.float64)
        e = C.c_double(0.0)
        v = np.zeros(6, np.float64)
        mx = C.c_int(0)
        _check(lib().ai2b_md_session_compute(self.h, C.c_int(nlocal), C.c_int(nghost), x.ctypes.data_as(C.c_void_p),
                                             t.ctypes.data_as(C.c_void_p), C.c_int(int(want_virial)), f.ctypes.data_as(C.c_void_p),
                                             C.byref(e), v.ctypes.data_as(C.c_void_p), C.byref(mx)))
        return e.value, f, v, mx.value

    def close(self):
        if self.h:
            lib().ai2b_md_session_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

