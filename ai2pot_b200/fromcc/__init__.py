"""Mirror of the reference's op loader ``ai2pot.fromcc`` (ai2pot/fromcc/__init__.py:52-134) for the
hot-path ops: loads the torch-op libraries built in ai2pot_b200/_lib (same file names as the
reference ships), points the MTP template search at ``ai2pot_path`` and re-exports the handles
under the reference's Python names.

    from ai2pot_b200 import fromcc
    fromcc.linearMtpToEFVOp(...), fromcc.nepToEFVOp(...), fromcc.forceSrOp(...), fromcc.nblist.find_info4mlff(...)

The dataset-statistics ops of the pre-training pass (fitutils) are provided too; ops outside the
per-atom evaluation path (deepmd, nnmtp, Gram/cross solver, Schmidt orthogonalisation) are not.
"""
import os

import torch

from . import nblist  # noqa: F401  (drop-in for the reference's CPython module of the same name)

_LIBDIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib")
ai2pot_path = os.environ.get("AI2POT_PATH", os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

for _name in ("libmtpr_bind.so", "libnep_bind.so", "libfvt_sr_op_bind.so", "libfitutils_bind.so"):
    _p = os.path.join(_LIBDIR, _name)
    if not os.path.exists(_p):
        raise ImportError(f"{_p} is missing: run `python -m ai2pot_b200._build` (there is no CPU fallback)")
    torch.ops.load_library(_p)

mtpParamOp = torch.ops.mtpr.mtpParamOp
linearMtpToEFVOp = torch.ops.mtpr.linearMtpToEFVOp
linearMtpToEFOp = torch.ops.mtpr.linearMtpToEFOp
linearMtpToDescriptorsOp = torch.ops.mtpr.linearMtpToDescriptorsOp
torch.ops.mtpr.set_ai2pot_path(ai2pot_path)

nepToEFOp = torch.ops.nep.nepToEFOp
nepToEFVOp = torch.ops.nep.nepToEFVOp
nepToDescriptorsOp = torch.ops.nep.nepToDescriptorsOp

forceSrOp = torch.ops.fvt.ForceSrOp
virialSrOp = torch.ops.fvt.VirialSrOp

targetStatisticsOp = torch.ops.fitutils.targetStatisticsOp
allTypeDescriptorsStatisticsOp = torch.ops.fitutils.allTypeDescriptorsStatisticsOp
eachTypeDescriptorsStatisticsOp = torch.ops.fitutils.eachTypeDescriptorsStatisticsOp
allTypeDescriptorsMaxminOp = torch.ops.fitutils.allTypeDescriptorsMaxminOp


linearMtpToLossOp = torch.ops.mtpr.linearMtpToLossOp
linearMtpToEFLossOp = torch.ops.mtpr.linearMtpToEFLossOp
nepToLossOp = torch.ops.nep.nepToLossOp
nepToEFLossOp = torch.ops.nep.nepToEFLossOp
