"""MTP training path on the GPU: loss, RMSEs and the analytic coefficient gradients against the
golden outputs of the reference's CPU code and against the CPU checkers (fp64 rel 1e-10)."""
import os
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(util.GOLDEN, "golden_small.npz"))


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _dev(g, nb, dt=torch.float64):
    prog = capi.MtpProgram(g["model"]["tables"])
    md = capi.to_device({k: v for k, v in g["model"].items() if k != "tables"}, float_dtype=dt)
    nbd = capi.to_device(nb)
    t = g["targets"]
    npad = nb["bilist"].shape[1]
    tg = [torch.from_numpy(np.ascontiguousarray(x)).to(dt).cuda() for x in (t["E"], t["F"][:, :npad], t["V"])]
    return prog, md, nbd, tg


def test_training_golden(checkers):
    g, nb = util.training_batch(_chk(checkers))
    prog, md, nbd, (E, F, V) = _dev(g, nb)
    e, f, v = capi.mtp_efv(prog, md, nbd)
    loss, rmse = capi.mtp_loss(nbd, g["weights"], e, E, f, F, v, V)
    assert util.relerr(loss.cpu().numpy(), G["train_loss"]) < 1e-10
    dco, dli, dbi = capi.mtp_loss_backward(prog, md, nbd, g["weights"], e, E, f, F, v, V)
    assert util.relerr(dco.cpu().numpy(), G["train_dcoeffs"]) < 1e-10
    assert util.relerr(dli.cpu().numpy(), G["train_dlinear"]) < 1e-10
    assert util.relerr(dbi.cpu().numpy(), G["train_dbias"]) < 1e-10
    # RMSE definitions of the op: sqrt(sum dE^2 / B), sqrt(sum dF^2 / (3 sum n)), sqrt(sum dV^2 / (9 B))
    en, fn_, vn = e.cpu().numpy(), f.cpu().numpy(), v.cpu().numpy()
    t = g["targets"]; npad = nb["bilist"].shape[1]; B = len(en)
    mask = (np.arange(npad)[None] < nb["binum"][:, None])[..., None]
    exp = [np.sqrt(((en - t["E"]) ** 2).sum() / B), np.sqrt((((fn_ - t["F"][:, :npad]) ** 2) * mask).sum() / (3 * nb["binum"].sum())),
           np.sqrt(((vn - t["V"]) ** 2).sum() / (9 * B))]
    assert util.relerr(rmse.cpu().numpy(), np.array(exp)) < 1e-12


@pytest.mark.parametrize("virial", [True, False])
def test_level16_batch_vs_checker(checkers, virial):
    """Level 16 (the training configuration's model) on a ragged batch with unequal weights."""
    chk = _chk(checkers)
    g, nb = util.training_batch(chk, level=16, B=4, seed=33, nmin=30, nmax=64)
    g["weights"] = (0.7, 1.3, 0.4)
    prog, md, nbd, (E, F, V) = _dev(g, nb)
    e, f, v = capi.mtp_efv(prog, md, nbd)
    en, fn_, vn = e.cpu().numpy(), f.cpu().numpy(), v.cpu().numpy()
    t = g["targets"]; npad = nb["bilist"].shape[1]
    if virial:
        loss, _ = capi.mtp_loss(nbd, g["weights"], e, E, f, F, v, V)
        got = capi.mtp_loss_backward(prog, md, nbd, g["weights"], e, E, f, F, v, V)
        lr = chk.mtp_loss(nb, g["weights"], en, t["E"], fn_, t["F"][:, :npad], vn, t["V"])
        ref = chk.mtp_loss_backward(g["model"], nb, g["weights"], en, t["E"], fn_, t["F"][:, :npad], vn, t["V"])
    else:
        loss, _ = capi.mtp_loss(nbd, g["weights"], e, E, f, F)
        got = capi.mtp_loss_backward(prog, md, nbd, g["weights"], e, E, f, F)
        lr = chk.mtp_loss(nb, g["weights"], en, t["E"], fn_, t["F"][:, :npad])
        ref = chk.mtp_loss_backward(g["model"], nb, g["weights"], en, t["E"], fn_, t["F"][:, :npad])
    assert util.relerr(loss.cpu().numpy(), lr) < 1e-10
    for a, b, name in zip(got, ref, ("coeffs", "linear", "bias")):
        assert util.relerr(a.cpu().numpy(), b) < 1e-10, name


def test_g3_full_batch_vs_checker(checkers):
    """configs[3] itself: 64 structures of 64-256 atoms, level 16, fp64. The padded neighbour tensors are built on the
    device in one launch (ai2b_nblist_build_batch) and must equal the CPU code's lists bit for bit; then E/F/V,
    loss[64], the three RMSEs and all three per-structure gradients against the CPU code at rel 1e-10."""
    chk = _chk(checkers)
    g = synth.g3(util.tables(16))
    structs = g["structs"]
    B = len(structs)
    npad = max(len(s["types"]) for s in structs)
    lists = []
    for s in structs:
        nn, fn, rc, ty, mx = chk.nblist(s["cell"], s["types"], s["coords"], g["rcut"], g["umax"])
        lists.append((nn, fn, rc, ty))
    nb = synth.pad_batch(lists, 3, g["umax"])
    coords = np.zeros((B, npad, 3)); binum = np.zeros(B, np.int32)
    for b, s in enumerate(structs):
        binum[b] = len(s["types"]); coords[b, :binum[b]] = s["coords"]
    cells = np.stack([s["cell"] for s in structs])
    nbd = capi.nblist_build_batch(cells, torch.from_numpy(binum).cuda(), torch.from_numpy(coords).cuda(), g["rcut"], g["umax"])
    st = nbd["status"].cpu().numpy()
    assert st[1] == 0 and st[0] == max(int(l[0].max()) for l in lists)
    assert np.array_equal(nbd["bilist"].cpu().numpy(), nb["bilist"])
    for b in range(B):
        n = binum[b]
        util.assert_nblist_equal((nbd["bnumneigh"][b, :n].cpu().numpy(), nbd["bfirstneigh"][b, :n].cpu().numpy(), nbd["brcs"][b, :n].cpu().numpy()),
                                 (lists[b][0], lists[b][1], lists[b][2]))
        assert int(nbd["bnumneigh"][b, n:].abs().sum()) == 0 and bool((nbd["bfirstneigh"][b, n:] == -1).all())
    nbd.update(btypes=torch.from_numpy(nb["btypes"]).cuda(), ntypes=3, nghost=0)
    prog, md, _, (E, F, V) = _dev(g, nb)
    e, f, v = capi.mtp_efv(prog, md, nbd)
    er, fr, vr = chk.mtp_efv(g["model"], nb)
    assert util.relerr(e.cpu().numpy(), er) < 1e-10 and util.relerr(f.cpu().numpy(), fr) < 1e-10 and util.relerr(v.cpu().numpy(), vr) < 1e-10
    t = g["targets"]
    loss, rmse = capi.mtp_loss(nbd, g["weights"], e, E, f, F, v, V)
    got = capi.mtp_loss_backward(prog, md, nbd, g["weights"], e, E, f, F, v, V)
    lr = chk.mtp_loss(nb, g["weights"], er, t["E"], fr, t["F"][:, :npad], vr, t["V"])
    ref = chk.mtp_loss_backward(g["model"], nb, g["weights"], er, t["E"], fr, t["F"][:, :npad], vr, t["V"])
    errs = dict(loss=util.relerr(loss.cpu().numpy(), lr))
    for a, r, name in zip(got, ref, ("dcoeffs", "dlinear", "dbias")):
        errs[name] = util.relerr(a.cpu().numpy(), r)
    mask = (np.arange(npad)[None] < binum[:, None])[..., None]
    exp = [np.sqrt(((er - t["E"]) ** 2).sum() / B), np.sqrt((((fr - t["F"][:, :npad]) ** 2) * mask).sum() / (3 * binum.sum())),
           np.sqrt(((vr - t["V"]) ** 2).sum() / (9 * B))]
    errs["rmse"] = util.relerr(rmse.cpu().numpy(), np.array(exp))
    print("configs[3] full batch, CUDA vs CPU code:", errs)
    assert max(errs.values()) < 1e-10, errs


def test_loss_op_autograd(checkers):
    """torch.ops.mtpr.linearMtpToLossOp: outputs and autograd gradients of mean(loss)."""
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    g, nb = util.training_batch(chk)
    m, tb, t = g["model"], g["model"]["tables"], g["targets"]
    npad = nb["bilist"].shape[1]; B = len(nb["binum"])
    dt = torch.float64
    c = lambda a, d=None: (torch.from_numpy(np.ascontiguousarray(a)).to(d) if d else torch.from_numpy(np.ascontiguousarray(a))).cuda()
    coeffs = c(m["coeffs"], dt).requires_grad_(True); lin = c(m["linear_coeffs"], dt).requires_grad_(True)
    bias = c(m["type_bias"], dt).requires_grad_(True)
    z = torch.zeros(36, dtype=dt, device="cuda")
    tail = (m["chebyshev_size"], m["scaling"], coeffs, lin, bias, tb["alpha_moments_count"], c(tb["alpha_index_basic"]),
            c(tb["alpha_index_times"]), c(tb["alpha_moment_mapping"]), tb["nmus"], c(nb["binum"]), c(nb["bilist"]), c(nb["bnumneigh"]),
            c(nb["bfirstneigh"]), c(nb["brcs"]), c(nb["btypes"]), torch.arange(3, dtype=torch.int32, device="cuda"), 0, m["rmax"], m["rmin"],
            c(m["q_scaler"], dt), 0.0, 0.0, z, z)
    loss, e_rmse, f_rmse, v_rmse = fromcc.linearMtpToLossOp(1.0, 1.0, 1.0, c(t["E"], dt), c(t["F"][:, :npad], dt),
                                                            c(t["V"].reshape(B, 3, 3), dt), *tail)
    assert util.relerr(loss.detach().cpu().numpy(), G["train_loss"]) < 1e-10 and e_rmse.shape == (1,)
    loss.mean().backward()
    assert util.relerr(coeffs.grad.cpu().numpy(), G["train_dcoeffs"].mean(0)) < 1e-10
    assert util.relerr(lin.grad.cpu().numpy(), G["train_dlinear"].mean(0)) < 1e-10
    assert util.relerr(bias.grad.cpu().numpy(), G["train_dbias"].mean(0)) < 1e-10
    out = fromcc.linearMtpToEFLossOp(1.0, 1.0, c(t["E"], dt), c(t["F"][:, :npad], dt), *tail)
    assert len(out) == 3
