"""agpt_b200: the trie-walk attention hot path of AGPT for NVIDIA B200 (sm_100a).

The compute lives in ``libagpt_b200.so`` (C ABI, ``include/agpt_b200.h``); this package is
the host-side mirror of the reference's operator interface on top of it.
"""
from ._lib import AgptError, lib  # noqa: F401
from .api import *  # noqa: F401,F403
