"""TEST INFRASTRUCTURE: ctypes bindings to the two CPU checkers.

* ``Checker("ref")``    -> oracle/_ref/libai2pot_ref.so, the reference's own CPU code
  (compiled from the reference tree by oracle/Makefile; see ref_driver.cc).
* ``Checker("oracle")`` -> oracle/_build/libai2pot_oracle.so, this repository's plain-C
  restatement of the same algorithms (oracle.c).

Both export the same functions with the prefixes ``ref_`` / ``orc_`` so one wrapper serves
both. Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
module; the shipped package never does.
"""
import ctypes as C
import os
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {"ref": ("_ref/libai2pot_ref.so", "ref_"), "oracle": ("_build/libai2pot_oracle.so", "orc_")}


def available(kind):
    return os.path.exists(os.path.join(_HERE, _LIBS[kind][0]))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _ci(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Checker:
    """Numpy-level access to one checker library. All arrays are host arrays; float dtype of
    ``brcs`` selects the f32/f64 entry point exactly as the reference ops do."""

    def __init__(self, kind="ref"):
        path, self.prefix = _LIBS[kind]
        self.kind = kind
        self.lib = C.CDLL(os.path.join(_HERE, path))

    def _fn(self, name, dtype):
        suf = "f64" if np.dtype(dtype) == np.float64 else "f32"
        f = getattr(self.lib, f"{self.prefix}{name}_{suf}")
        f.restype = C.c_int
        return f, (C.c_double if suf == "f64" else C.c_float)

    # -- neighbour list ---------------------------------------------------------------
    def nblist(self, cell, types, coords, rcut, umax, is_cart=True, pbc=(1, 1, 1), sort=False):
        dt = coords.dtype
        f, _ = self._fn("nblist", dt)
        n = coords.shape[0]
        cell = np.ascontiguousarray(cell, dtype=dt)
        coords = np.ascontiguousarray(coords)
        types = _ci(types)
        pbc = _ci(pbc)
        numneigh = np.zeros(n, np.int32)
        first = np.zeros((n, umax), np.int32)
        rcs = np.zeros((n, umax, 3), dt)
        tout = np.zeros(n, np.int32)
        mx = C.c_int(0)
        rc = f(C.c_int(n), _p(cell), _p(types), _p(coords), C.c_int(int(is_cart)), C.c_double(rcut),
               _p(pbc), C.c_int(int(sort)), C.c_int(umax), _p(numneigh), _p(first), _p(rcs), _p(tout),
               C.byref(mx))
        if rc != 0:
            raise RuntimeError(f"nblist: max neighbours {mx.value} > umax {umax}")
        return numneigh, first, rcs, tout, mx.value

    # -- .almtp parsing (reference only) ------------------------------------------------
    def mtp_param_file(self, filename):
        f = getattr(self.lib, self.prefix + "mtp_param_file")
        f.restype = C.c_int
        counts = np.zeros(5, np.int32)
        if f(filename.encode(), _p(counts), None, None, None) != 0:
            raise RuntimeError("cannot parse " + filename)
        basic = np.zeros((counts[1], 4), np.int32)
        times = np.zeros((counts[2], 4), np.int32)
        mapping = np.zeros(counts[3], np.int32)
        f(filename.encode(), _p(counts), _p(basic), _p(times), _p(mapping))
        return dict(alpha_moments_count=int(counts[0]), alpha_index_basic=basic, alpha_index_times=times,
                    alpha_moment_mapping=mapping, nmus=int(counts[4]))

    # -- helpers ------------------------------------------------------------------------
    @staticmethod
    def _tab(tb):
        return (C.c_int(tb["alpha_moments_count"]), C.c_int(len(tb["alpha_index_basic"])),
                _p(_ci(tb["alpha_index_basic"])), C.c_int(len(tb["alpha_index_times"])),
                _p(_ci(tb["alpha_index_times"])), C.c_int(len(tb["alpha_moment_mapping"])),
                _p(_ci(tb["alpha_moment_mapping"])), C.c_int(tb["nmus"]))

    @staticmethod
    def _nb(nb, keep):
        B, Np = nb["bilist"].shape
        umax = nb["bfirstneigh"].shape[2]
        arrs = [_ci(nb["binum"]), _ci(nb["bilist"]), _ci(nb["bnumneigh"]), _ci(nb["bfirstneigh"]),
                np.ascontiguousarray(nb["brcs"]), _ci(nb["btypes"]), _ci(np.arange(nb["ntypes"]))]
        keep.extend(arrs)
        return (C.c_int(B), C.c_int(Np), _p(arrs[0]), _p(arrs[1]), _p(arrs[2]), _p(arrs[3]), _p(arrs[4]),
                _p(arrs[5]), C.c_int(nb["ntypes"]), _p(arrs[6]), C.c_int(umax), C.c_int(nb.get("nghost", 0)))

    # -- linear MTP -----------------------------------------------------------------------
    def mtp_efv(self, model, nb, virial=True):
        dt = nb["brcs"].dtype
        f, cf = self._fn("mtp_efv" if virial else "mtp_ef", dt)
        B, Np = nb["bilist"].shape
        ng = nb.get("nghost", 0)
        e = np.zeros(B, dt); frc = np.zeros((B, Np + ng, 3), dt); vir = np.zeros((B, 9), dt)
        keep = []
        par = [np.ascontiguousarray(model[k], dtype=dt) for k in ("coeffs", "linear_coeffs", "type_bias", "q_scaler")]
        out = (_p(e), _p(frc), _p(vir)) if virial else (_p(e), _p(frc))
        f(*out, C.c_int(model["chebyshev_size"]), cf(model["scaling"]), _p(par[0]), _p(par[1]), _p(par[2]),
          *self._tab(model["tables"]), *self._nb(nb, keep), cf(model["rmax"]), cf(model["rmin"]), _p(par[3]))
        return (e, frc, vir) if virial else (e, frc)

    def mtp_descriptors(self, model, nb):
        dt = nb["brcs"].dtype
        f, cf = self._fn("mtp_descriptors", dt)
        B, Np = nb["bilist"].shape
        ns = len(model["tables"]["alpha_moment_mapping"])
        d = np.zeros((B, Np, ns), dt)
        keep = []
        co = np.ascontiguousarray(model["coeffs"], dtype=dt)
        f(_p(d), C.c_int(model["chebyshev_size"]), cf(model["scaling"]), _p(co), *self._tab(model["tables"]),
          *self._nb(nb, keep), cf(model["rmax"]), cf(model["rmin"]))
        return d

    def mtp_loss(self, nb, w, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
        dt = nb["brcs"].dtype
        B, Np = nb["bilist"].shape
        loss = np.zeros(B, dt)
        a = [_ci(nb["binum"]), _ci(nb["bilist"])] + [np.ascontiguousarray(x, dtype=dt) for x in (e_ml, e_dft, f_ml, f_dft)]
        if v_ml is not None:
            f, cf = self._fn("mtp_loss", dt)
            v = [np.ascontiguousarray(x, dtype=dt) for x in (v_ml, v_dft)]
            f(_p(loss), C.c_int(B), C.c_int(Np), _p(a[0]), _p(a[1]), cf(w[0]), cf(w[1]), cf(w[2]), _p(a[2]), _p(a[3]),
              _p(a[4]), _p(a[5]), _p(v[0]), _p(v[1]))
        else:
            f, cf = self._fn("mtp_ef_loss", dt)
            f(_p(loss), C.c_int(B), C.c_int(Np), _p(a[0]), _p(a[1]), cf(w[0]), cf(w[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(a[5]))
        return loss

    def mtp_loss_backward(self, model, nb, w, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
        """Per-structure gradients [B,num_coeffs], [B,n_scalar], [B,ntypes]."""
        dt = nb["brcs"].dtype
        B, Np = nb["bilist"].shape
        tb = model["tables"]
        dco = np.zeros((B, model["coeffs"].size), dt)
        dli = np.zeros((B, len(tb["alpha_moment_mapping"])), dt)
        dbi = np.zeros((B, nb["ntypes"]), dt)
        keep = []
        par = [np.ascontiguousarray(model[k], dtype=dt) for k in ("coeffs", "linear_coeffs", "type_bias", "q_scaler")]
        a = [np.ascontiguousarray(x, dtype=dt) for x in (e_ml, e_dft, f_ml, f_dft)]
        if v_ml is not None:
            f, cf = self._fn("mtp_loss_backward", dt)
            v = [np.ascontiguousarray(x, dtype=dt) for x in (v_ml, v_dft)]
            f(_p(dco), _p(dli), _p(dbi), cf(w[0]), cf(w[1]), cf(w[2]), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(v[0]), _p(v[1]),
              C.c_int(model["chebyshev_size"]), cf(model["scaling"]), _p(par[0]), _p(par[1]), _p(par[2]),
              *self._tab(tb), *self._nb(nb, keep), cf(model["rmax"]), cf(model["rmin"]), _p(par[3]))
        else:
            f, cf = self._fn("mtp_ef_loss_backward", dt)
            f(_p(dco), _p(dli), _p(dbi), cf(w[0]), cf(w[1]), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]),
              C.c_int(model["chebyshev_size"]), cf(model["scaling"]), _p(par[0]), _p(par[1]), _p(par[2]),
              *self._tab(tb), *self._nb(nb, keep), cf(model["rmax"]), cf(model["rmin"]), _p(par[3]))
        return dco, dli, dbi

    # -- NEP ------------------------------------------------------------------------------
    def nep_efv(self, model, nb, virial=True):
        dt = nb["brcs"].dtype
        f, cf = self._fn("nep_efv" if virial else "nep_ef", dt)
        B, Np = nb["bilist"].shape
        ng = nb.get("nghost", 0)
        e = np.zeros(B, dt); frc = np.zeros((B, Np + ng, 3), dt); vir = np.zeros((B, 9), dt)
        keep = []
        par = [np.ascontiguousarray(model[k], dtype=dt) for k in ("coeffs", "w0", "b0", "w1", "type_bias", "q_scaler")]
        out = (_p(e), _p(frc), _p(vir)) if virial else (_p(e), _p(frc))
        f(*out, C.c_int(model["chebyshev_size"]), C.c_int(model["n_radial"]), C.c_int(model["n_angular"]),
          C.c_int(model["l_max"]), C.c_int(model["num_neurons"]), *[_p(x) for x in par[:5]],
          *self._nb(nb, keep), cf(model["rmax_radial"]), cf(model["rmax_angular"]), _p(par[5]))
        return (e, frc, vir) if virial else (e, frc)

    def nep_loss_backward(self, model, nb, w, e_ml, e_dft, f_ml, f_dft, v_ml=None, v_dft=None):
        """Per-structure gradients [B,num_coeffs], [B,ntypes*neurons*nd], [B,ntypes*neurons] (b0, w1), [B,ntypes]."""
        dt = nb["brcs"].dtype
        B, Np = nb["bilist"].shape
        nt, nneu = nb["ntypes"], model["num_neurons"]
        nd = model["n_radial"] + model["n_angular"] * model["l_max"]
        dco = np.zeros((B, model["coeffs"].size), dt); dw0 = np.zeros((B, nt * nneu * nd), dt)
        db0 = np.zeros((B, nt * nneu), dt); dw1 = np.zeros((B, nt * nneu), dt); dbi = np.zeros((B, nt), dt)
        keep = []
        par = [np.ascontiguousarray(model[k], dtype=dt) for k in ("coeffs", "w0", "b0", "w1", "type_bias", "q_scaler")]
        a = [np.ascontiguousarray(x, dtype=dt) for x in (e_ml, e_dft, f_ml, f_dft)]
        mdl = (C.c_int(model["chebyshev_size"]), C.c_int(model["n_radial"]), C.c_int(model["n_angular"]), C.c_int(model["l_max"]),
               C.c_int(nneu), *[_p(x) for x in par[:5]])
        if v_ml is not None:
            f, cf = self._fn("nep_loss_backward", dt)
            v = [np.ascontiguousarray(x, dtype=dt) for x in (v_ml, v_dft)]
            f(_p(dco), _p(dw0), _p(db0), _p(dw1), _p(dbi), cf(w[0]), cf(w[1]), cf(w[2]), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]),
              _p(v[0]), _p(v[1]), *mdl, *self._nb(nb, keep), cf(model["rmax_radial"]), cf(model["rmax_angular"]), _p(par[5]))
        else:
            f, cf = self._fn("nep_ef_loss_backward", dt)
            f(_p(dco), _p(dw0), _p(db0), _p(dw1), _p(dbi), cf(w[0]), cf(w[1]), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]),
              *mdl, *self._nb(nb, keep), cf(model["rmax_radial"]), cf(model["rmax_angular"]), _p(par[5]))
        return dco, dw0, db0, dw1, dbi

    def nep_descriptors(self, model, nb):
        dt = nb["brcs"].dtype
        f, cf = self._fn("nep_descriptors", dt)
        B, Np = nb["bilist"].shape
        nd = model["n_radial"] + model["n_angular"] * model["l_max"]
        d = np.zeros((B, Np, nd), dt)
        keep = []
        co = np.ascontiguousarray(model["coeffs"], dtype=dt)
        f(_p(d), C.c_int(model["chebyshev_size"]), C.c_int(model["n_radial"]), C.c_int(model["n_angular"]),
          C.c_int(model["l_max"]), _p(co), *self._nb(nb, keep), cf(model["rmax_radial"]), cf(model["rmax_angular"]))
        return d

    # -- fvt (values) ---------------------------------------------------------------------
    def fvt_force(self, ilist, numneigh, firstneigh, nghost, dei_drij):
        dt = dei_drij.dtype
        f, _ = self._fn("fvt_force", dt)
        inum, umax = firstneigh.shape
        out = np.zeros((inum + nghost, 3), dt)
        a = [_ci(ilist), _ci(numneigh), _ci(firstneigh), np.ascontiguousarray(dei_drij)]
        f(_p(out), C.c_int(inum), _p(a[0]), _p(a[1]), _p(a[2]), C.c_int(nghost), C.c_int(umax), _p(a[3]))
        return out

    def fvt_virial(self, numneigh, rcs, dei_drij):
        dt = dei_drij.dtype
        f, _ = self._fn("fvt_virial", dt)
        inum, umax = rcs.shape[:2]
        out = np.zeros(9, dt)
        a = [_ci(numneigh), np.ascontiguousarray(rcs), np.ascontiguousarray(dei_drij)]
        f(_p(out), C.c_int(inum), _p(a[0]), _p(a[1]), C.c_int(umax), _p(a[2]))
        return out

    # -- ZBL pair correction (accumulates into copies of e, f, v) ---------------------------
    def zbl(self, nb1, type_map, rmax, rmin, cks, dks, e=0.0, f=None, v=None, variant="efv"):
        """One structure: nb1 = dict(ilist, numneigh, firstneigh, rcs, types, nghost). variant "efv" is the
        complete correction (energy, centre-atom force, virial); "cpu_efv" / "cpu_ef" are the reference's
        CPU group calls (reference build only)."""
        rcs = np.ascontiguousarray(nb1["rcs"])
        dt = rcs.dtype
        fn, _ = self._fn("zbl_" + variant, dt)
        inum, umax = nb1["firstneigh"].shape
        ng = int(nb1.get("nghost", 0))
        eo = np.array([e], dt)
        fo = np.zeros((inum + ng, 3), dt) if f is None else np.array(f, dt).reshape(inum + ng, 3).copy()
        vo = np.zeros(9, dt) if v is None else np.array(v, dt).reshape(9).copy()
        a = [_ci(nb1["ilist"]), _ci(nb1["numneigh"]), _ci(nb1["firstneigh"]), rcs, _ci(nb1["types"]), _ci(type_map),
             np.ascontiguousarray(cks, dt), np.ascontiguousarray(dks, dt)]
        ct = C.c_double if dt == np.float64 else C.c_float
        ntypes = len(type_map)
        if variant == "cpu_ef":
            fn(_p(eo), _p(fo), C.c_int(inum), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), C.c_int(ntypes), _p(a[5]),
               C.c_int(umax), C.c_int(ng), ct(rmax), ct(rmin), _p(a[6]), _p(a[7]))
        else:
            fn(_p(eo), _p(fo), _p(vo), C.c_int(inum), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), C.c_int(ntypes),
               _p(a[5]), C.c_int(umax), C.c_int(ng), ct(rmax), ct(rmin), _p(a[6]), _p(a[7]))
        return eo[0], fo, vo

    # -- dataset statistics -------------------------------------------------------------------
    def desc_stats(self, binum, bdesc, bilist=None, btypes=None, ntypes=1):
        dt = bdesc.dtype
        B, npad, nd = bdesc.shape
        each = btypes is not None
        n = np.zeros(ntypes if each else 1, np.int32)
        mean = np.zeros((ntypes, nd) if each else nd, dt); m2 = np.zeros_like(mean)
        d = np.ascontiguousarray(bdesc); bn = _ci(binum)
        if each:
            f, _ = self._fn("desc_stats_each", dt)
            bl, bt = _ci(bilist), _ci(btypes)
            f(_p(n), _p(mean), _p(m2), C.c_int(B), C.c_int(npad), C.c_int(nd), _p(bn), _p(bl), _p(bt), C.c_int(ntypes), _p(d))
        else:
            f, _ = self._fn("desc_stats_all", dt)
            f(_p(n), _p(mean), _p(m2), C.c_int(B), C.c_int(npad), C.c_int(nd), _p(bn), _p(d))
        return n, mean, m2

    def desc_maxmin(self, binum, bdesc):
        dt = bdesc.dtype
        B, npad, nd = bdesc.shape
        mx = np.zeros(nd, dt); mn = np.zeros(nd, dt)
        f, _ = self._fn("desc_maxmin", dt)
        d = np.ascontiguousarray(bdesc); bn = _ci(binum)
        f(_p(mx), _p(mn), C.c_int(B), C.c_int(npad), C.c_int(nd), _p(bn), _p(d))
        return mx, mn

    def target_stats(self, binum, etot, force):
        dt = etot.dtype
        B, npad = force.shape[:2]
        n = np.zeros(1, np.int32); out = np.zeros(3, dt)
        f, _ = self._fn("target_stats", dt)
        e = np.ascontiguousarray(etot); fo = np.ascontiguousarray(force); bn = _ci(binum)
        f(_p(n), _p(out), C.c_int(B), C.c_int(npad), _p(bn), _p(e), _p(fo))
        return int(n[0]), out

