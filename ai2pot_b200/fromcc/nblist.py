"""Drop-in for the reference's CPython module ``nblist`` (source/nblist/bind/nblist_bind.cc:35-207),
backed by the CUDA cell-list builder through the C ABI.

    find_info4mlff(cell, types, coords, rcut, umax, is_cart, pbc, sort)
        -> (inum, ilist, numneigh, firstneigh, rcs, types, nghost)

Same argument order, dtypes (float32 / float64 selected by ``coords``; int64 types are narrowed to
int32) and return tuple as the reference. TypeError on wrong Python types, like the reference;
a row longer than ``umax`` raises (the reference silently overruns its buffer there).
"""
import numpy as np
import torch

from .. import capi

_builder = None


def find_info4mlff(cell, types, coords, rcut, umax, is_cart, pbc, sort):
    global _builder
    if not isinstance(cell, np.ndarray) or not isinstance(types, np.ndarray) or not isinstance(coords, np.ndarray):
        raise TypeError("cell, types and coords must be numpy arrays")
    if not isinstance(pbc, (list, tuple)) or len(pbc) != 3:
        raise TypeError("pbc must be a list of three bools")
    if coords.dtype not in (np.float32, np.float64) or cell.dtype != coords.dtype:
        raise TypeError("cell and coords must both be float32 or both float64")
    if types.dtype not in (np.int32, np.int64):
        raise TypeError("types must be int32 or int64")
    n = int(coords.shape[0])
    if _builder is None:
        _builder = capi.NeighborBuilder()
    dcoords = torch.from_numpy(np.ascontiguousarray(coords)).cuda()
    nn, fn, rcs, status = _builder.build(cell, dcoords, float(rcut), int(umax), bool(is_cart), pbc)
    if sort:
        nn, fn, rcs = capi.sort_rows_by_distance(nn, fn, rcs)
    st = status.cpu().numpy()
    if st[1]:
        raise ValueError(f"umax={umax} is smaller than the largest neighbour count {int(st[0])}")
    return (n, np.arange(n, dtype=np.int32), nn.cpu().numpy(), fn.cpu().numpy(), rcs.cpu().numpy(),
            np.ascontiguousarray(types, dtype=np.int32), 0)
