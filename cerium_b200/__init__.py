"""cerium_b200: B200-native RNS-CKKS evaluation core behind a C ABI (include/cerium_b200.h)."""
from . import params  # noqa: F401
from ._capi import (BCONV_EXACT, BCONV_LAZY, ROUND_FLOOR, ROUND_HALF, BaseConverter, CeriumError, Context,  # noqa: F401
                    KeySwitch, Library, load)

__all__ = ["params", "Library", "Context", "BaseConverter", "KeySwitch", "CeriumError", "load",
           "BCONV_LAZY", "BCONV_EXACT", "ROUND_FLOOR", "ROUND_HALF"]
