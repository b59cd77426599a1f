"""ai2b_nep_efv_static_scratch_f32: the NEP entry point for hosts that cannot allocate device
memory (an MD loop that must not stall the device, a program whose memory belongs to its own
pool). It keeps its scratch in an array inside the library instead of taking a workspace.

Called through the C ABI twice in a row, on two different systems and models, and compared with
ai2b_nep_efv_f32 (caller-owned workspace) on the same inputs within the fp32 tolerance of the NEP
parity tests (1e-5 of the tensor's scale; the two differ only by the order of atomic sums).
Collected last, so a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth
from oracle import refapi

pytestmark = pytest.mark.gpu


def _inputs(seed, n, ntypes, **cfg):
    rng = np.random.default_rng(seed)
    cell, pos = synth.cubic_lattice(n, 3.0, 0.1, rng, np.float32)
    types = rng.integers(0, ntypes, len(pos)).astype(np.int32)
    model = synth.nep_model(ntypes, rng, np.float32, **cfg)
    chk = refapi.Checker("oracle")      # only builds the neighbour list the two entry points share
    nn, fm, rc, ty, mx = chk.nblist(cell, types, pos, model["rmax_radial"], 96)
    return capi.to_device(model), capi.to_device(synth.batch_from_nblist(nn, fm, rc, ty, ntypes))


def _static(model, nb):
    B, npad = nb["bilist"].shape
    umax = nb["bfirstneigh"].shape[2]
    e = torch.empty(B, dtype=torch.float32, device="cuda")
    f = torch.empty(B, npad, 3, dtype=torch.float32, device="cuda")
    v = torch.empty(B, 9, dtype=torch.float32, device="cuda")
    p = capi._ptr
    rc = capi.lib().ai2b_nep_efv_static_scratch_f32(
        p(e), p(f), p(v), C.c_int(model["chebyshev_size"]), C.c_int(model["n_radial"]), C.c_int(model["n_angular"]),
        C.c_int(model["l_max"]), C.c_int(model["num_neurons"]), p(model["coeffs"]), p(model["w0"]), p(model["b0"]), p(model["w1"]),
        p(model["type_bias"]), C.c_int(B), C.c_int(npad), p(nb["binum"]), p(nb["bilist"]), p(nb["bnumneigh"]), p(nb["bfirstneigh"]),
        p(nb["brcs"]), p(nb["btypes"]), C.c_int(nb["ntypes"]), C.c_int(umax), C.c_int(0), C.c_float(model["rmax_radial"]),
        C.c_float(model["rmax_angular"]), p(model["q_scaler"]), capi._stream())
    return rc, (e, f, v)


def test_static_scratch_matches_workspace_entry_twice():
    cases = [_inputs(101, 6, 3), _inputs(202, 5, 2, n_radial=6, n_angular=3, l_max=3, chebyshev_size=10, num_neurons=12)]
    for model, nb in cases:                  # two calls in a row share the built-in array
        rc, got = _static(model, nb)
        assert rc == 0, capi.lib().ai2b_last_error_string()
        want = capi.nep_efv(model, nb)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert util.relerr(a.cpu().numpy(), b.cpu().numpy()) < 1e-5
        assert float(got[1].abs().max()) > 0


def test_static_scratch_rejects_oversized_requests():
    model, nb = _inputs(303, 3, 2)
    big = dict(model, n_radial=4000)         # coefficient table far beyond 128 KiB; refused before any launch
    rc, _ = _static(big, nb)
    assert rc == -4 and b"131072" in capi.lib().ai2b_last_error_string()
