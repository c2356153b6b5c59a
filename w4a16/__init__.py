"""Drop-in alias: ``import w4a16`` resolves to the B200 implementation in ``nibble_b200``.

Module names mirror the reference package (``w4a16.cuda``, ``w4a16.linear``, ``w4a16.quantization``,
``w4a16.integration``, ``w4a16.checkpoint``).  The reference's CPU test routine ``w4a16.reference``
is deliberately not part of this package.
"""
from nibble_b200 import *  # noqa: F401,F403
from nibble_b200 import __all__  # noqa: F401
