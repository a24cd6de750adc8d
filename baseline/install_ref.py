"""Places an unmodified copy of the reference project under baseline/_ref/ (git-ignored).

The reference is a single module, `flash_attention.py`, with no setup.py / pyproject.toml, so
`pip install --target baseline/_ref <reference>` answers "not installable"; its one file is
therefore copied byte for byte.  The copy never enters the history (baseline/_ref/ is listed
in .gitignore) but travels with the working tree to a GPU machine, where the tests and
`bench.py --impl triton_ref` import it to run the reference's own Triton kernels on the
same inputs as this library.

    python baseline/install_ref.py [path/to/reference]
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def install(src_dir: str) -> str:
    src = os.path.join(src_dir, "flash_attention.py")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(DEST, exist_ok=True)
    dst = os.path.join(DEST, "flash_attention.py")
    shutil.copyfile(src, dst)
    with open(dst, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        f.write(f"unmodified copy of {src}\nsha256 {digest}\n")
    return dst


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
