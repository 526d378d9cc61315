"""Install the unmodified reference (latkins/trifast) into ``baseline/_ref`` (git-ignored).

    python baseline/install_ref.py /path/to/reference

The reference is a pure-Python package built with hatchling, which is not available
offline, so ``pip install --target baseline/_ref`` cannot run; this script does what that
install would: it copies ``src/trifast`` as it is and writes the ``dist-info`` metadata the
package reads its version from (``importlib.metadata.version("trifast")``,
src/trifast/autotune_helpers.py:24).  Nothing is edited.  The copy is used only by
``baseline/triton_ref.py`` (the same-GPU Triton measurement); the product never imports it.
"""

import os
import re
import shutil
import sys


def main(ref_root):
    here = os.path.dirname(os.path.abspath(__file__))
    dst = os.path.join(here, "_ref")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(os.path.join(ref_root, "src", "trifast"), os.path.join(dst, "trifast"),
                    ignore=shutil.ignore_patterns("__pycache__"))
    text = open(os.path.join(ref_root, "pyproject.toml")).read()
    version = re.search(r'^version\s*=\s*"([^"]+)"', text, re.M).group(1)
    info = os.path.join(dst, f"trifast-{version}.dist-info")
    os.makedirs(info)
    with open(os.path.join(info, "METADATA"), "w") as f:
        f.write(f"Metadata-Version: 2.1\nName: trifast\nVersion: {version}\n")
    with open(os.path.join(info, "RECORD"), "w") as f:
        f.write("")
    with open(os.path.join(info, "INSTALLER"), "w") as f:
        f.write("baseline/install_ref.py\n")
    print(f"installed trifast {version} into {dst}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: install_ref.py <path to a checkout of latkins/trifast>")
    main(sys.argv[1])
