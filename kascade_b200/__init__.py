"""kascade_b200 — B200 (sm_100a) implementation of the Kascade sparse-attention hot path.

``EfficientKascadeStrategy`` is the drop-in for the reference's strategy of the same name; the
kernels live in ``libkascade_b200.so`` (C ABI in ``include/kascade_b200.h``), built in-tree by
``python -m kascade_b200.build``.
"""
from .strategy import EfficientKascadeStrategy, Strategy, topk_budget  # noqa: F401

__version__ = "0.1.0"
