"""Regenerates ai2pot_b200/data/mtp_tables_L{06,10,16}.npz.

The alpha tables are parsed from the reference tree's template files BY THE REFERENCE'S OWN
PARSER (oracle/_ref, built by oracle/Makefile) and stored as int32 arrays. Run in a container
that has the reference mounted:  REF_ROOT=<reference tree> python ai2pot_b200/data/make_mtp_tables.py
"""
import os, sys
import numpy as np
sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle.refapi import Checker

root = sys.argv[1] if len(sys.argv) > 1 else os.environ["REF_ROOT"]
ref = Checker("ref")
for level in (6, 10, 16):
    t = ref.mtp_param_file(f"{root}/source/descriptor/mtpr/MTP_templates/{level:02d}.almtp")
    out = os.path.join(os.path.dirname(__file__), f"mtp_tables_L{level:02d}.npz")
    np.savez_compressed(out, alpha_moments_count=np.int32(t["alpha_moments_count"]), nmus=np.int32(t["nmus"]),
                        alpha_index_basic=t["alpha_index_basic"], alpha_index_times=t["alpha_index_times"],
                        alpha_moment_mapping=t["alpha_moment_mapping"])
    print(level, out, os.path.getsize(out))
