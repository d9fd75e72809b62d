"""The native all-to-all context (see csrc/a2a/a2a_context.h).
Same name as the reference's python/pplx_garden/native/p2p_all_to_all.py:3-5."""

from pplx_garden._native import AllToAllContext as AllToAllContext
