"""In-tree build of libteeny_b200.so (nvcc, sm_100a only)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def library_path():
    """The library the package loads: TEENY_B200_LIB if set (e.g. a -DTEENY_TRACE build made beside the default one),
    else the in-tree default build."""
    return os.environ.get("TEENY_B200_LIB") or os.path.join(_HERE, "libteeny_b200.so")


def build(force=False, jobs=8, verbose=False):
    """Compile every CUDA source for sm_100a (``make -C csrc``).  Cross-compiles without a GPU."""
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), f"-j{jobs}"]
    if force:
        cmd.append("-B")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
        print(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("building libteeny_b200.so failed")
    return library_path()
