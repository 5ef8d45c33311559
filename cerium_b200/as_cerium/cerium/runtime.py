"""``cerium.runtime`` (cerium/python/runtime/wrapper.cpp:62-235) re-exported from cerium_b200.runtime."""
from cerium_b200.runtime import (CeriumFunctionExecutor, Ciphertext, CKKSEncryptor, CKKSEncryptorContext,  # noqa: F401
                                 Context, FusedKernelProgram, IOGenerator, RawInputsWrapper)

__version__ = "cerium_b200"
