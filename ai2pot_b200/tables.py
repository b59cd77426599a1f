"""MTP alpha tables shipped with the package (ai2pot_b200/data/mtp_tables_LNN.npz): the int32 arrays the
reference's parser reads from its template files NN.almtp (source/descriptor/mtpr/src/mtpParam.cc:64-200), stored for
the levels the benchmark configurations use. Any other level is parsed from a template file with
``ai2pot_b200.capi.parse_almtp``."""
import os

import numpy as np

_DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")
LEVELS = (6, 10, 16)


def load(level):
    path = os.path.join(_DATA, f"mtp_tables_L{int(level):02d}.npz")
    if not os.path.exists(path):
        raise FileNotFoundError(f"no stored tables for MTP level {level} (stored: {LEVELS}); parse the template with capi.parse_almtp")
    z = np.load(path)
    return dict(alpha_moments_count=int(z["alpha_moments_count"]), nmus=int(z["nmus"]),
                alpha_index_basic=z["alpha_index_basic"], alpha_index_times=z["alpha_index_times"],
                alpha_moment_mapping=z["alpha_moment_mapping"])
