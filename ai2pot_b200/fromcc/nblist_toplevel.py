"""Top-level module ``nblist``: what the reference's loader finds after ``sys.path.append(lib_dir); import nblist``
(ai2pot/fromcc/__init__.py:52-58) when ``lib_dir`` is this build's ``ai2pot_b200/_lib``. The build step copies this
file there as ``nblist.py``. It re-exports the CUDA-backed ``find_info4mlff`` of ``ai2pot_b200.fromcc.nblist``
(same arguments and 7-tuple as source/nblist/bind/nblist_bind.cc:35-207)."""
import os
import sys

try:
    from ai2pot_b200.fromcc.nblist import find_info4mlff  # noqa: F401
except ImportError:
    # the package sits two directories above ai2pot_b200/_lib/nblist.py
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from ai2pot_b200.fromcc.nblist import find_info4mlff  # noqa: F401
