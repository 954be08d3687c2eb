"""Where the C-ABI library lives and how it is built (in-tree, for sm_100a)."""
import os
import subprocess

version = "0.1.0"

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PACKAGE_DIR)                       # metal-linalg_b200/
LIBRARY = os.path.join(ROOT, "lib", "libmetal_linalg.so")


def build(verbose=False):
    """Compiles every CUDA source for sm_100a into lib/libmetal_linalg.so (nvcc; no GPU needed)."""
    out = None if verbose else subprocess.DEVNULL
    subprocess.run(["make", "-C", ROOT, "-j", str(min(8, os.cpu_count() or 1))], check=True, stdout=out)
    return LIBRARY
