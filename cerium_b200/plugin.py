"""Installs the library as the kernel plugin of a compiled Cerium function.

The Cerium runtime loads ``<dir>/function_map_<p>.so`` for every partition ``p`` of a compiled
function (``cerium/runtime/execution/function.cpp:144-177``).  ``install(dir)`` puts one COPY of
``function_map_shim.so`` under each of those names - the generated plugin, when there is one, is
kept beside it as ``function_map_<p>.orig.so`` and still serves the element-wise records - so that
the ntt / int / sud / bco records of ``functions<p>`` run on this library's kernels.  Copies, not
links: the runtime loads all partitions into one process and links to one file would be folded
into a single loaded object.

    python -m cerium_b200.plugin <dir>/<function>
"""
from __future__ import annotations

import os
import re
import shutil
import sys
from typing import List

from . import build as _build


def partitions(function_dir: str) -> List[str]:
    """Partition ids that have a records file ``functions<p>`` in the directory."""
    out = []
    for name in sorted(os.listdir(function_dir)):
        m = re.fullmatch(r"functions(\d+)", name)
        if m:
            out.append(m.group(1))
    return out


def install(function_dir: str) -> List[str]:
    """Returns the plugin paths written."""
    if not os.path.exists(_build.SHIM_LIB):
        _build.build()
    written = []
    with open(_build.SHIM_LIB, "rb") as f:
        shim = f.read()
    for p in partitions(function_dir):
        dst = os.path.join(function_dir, "function_map_%s.so" % p)
        orig = os.path.join(function_dir, "function_map_%s.orig.so" % p)
        if os.path.lexists(dst):
            with open(dst, "rb") as f:
                same = f.read() == shim
            if same and not os.path.islink(dst):
                written.append(dst)
                continue
            if not os.path.exists(orig) and not os.path.islink(dst):
                os.rename(dst, orig)          # the generated plugin
            else:
                os.remove(dst)
        shutil.copyfile(_build.SHIM_LIB, dst)
        os.chmod(dst, 0o755)
        written.append(dst)
    return written


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    for path in install(sys.argv[1]):
        print(path)
