"""insignia_b200: sm_100a decode kernels + host classes for the Insignia token loop.

The product is ``lib/libinsignia_b200.so`` (C ABI: include/insignia_b200.h, C++ host
API: include/insignia_*.hpp).  The Python modules are callers of that ABI
(:mod:`ops`, :mod:`engine`) and host-side file utilities (:mod:`mxfp4`,
:mod:`checkpoint_io`, :mod:`synth`).
"""
__all__ = ["build", "checkpoint_io", "engine", "mxfp4", "ops", "synth"]
