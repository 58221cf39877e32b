"""Build recipe of the CUDA library: one nvcc call, sm_100a only, in-tree output."""

from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["gd_render.cu"]
HEADERS = ["gd_device.cuh", "gd_geometry.cuh", "gd_walk.cuh", "gd_flats.cuh", "gd_sprites.cuh", "gd_decals.cuh", "gd_output.cuh", "gd_abi.cuh", "gd_state.cuh", "gd_state_abi.cuh", "gd_move.cuh",
           "../../include/gradoom_b200.h", "../../include/gradoom_b200_layout.h"]
LIBRARY = os.path.join(HERE, "libgradoom_b200.so")
# the same sources with -DGD_CHECKED: every index taken from the blob or a record is range-tested
CHECKED_LIBRARY = os.path.join(HERE, "libgradoom_b200_checked.so")

# -fmad=false: the reference rounds every float32 multiply and add separately;
# a fused multiply-add would change texel and ownership decisions.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-fmad=false", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources_hash() -> str:
    """SHA-256 over the kernel sources and the two headers, in a fixed order: profile
    summaries are stamped with it so that a figure measured on other code is not quoted."""

    import hashlib

    digest = hashlib.sha256()
    for name in sorted(SOURCES + HEADERS):
        with open(os.path.join(HERE, name), "rb") as f:
            digest.update(name.encode() + b"\0" + f.read())
    return digest.hexdigest()


def is_stale(library: str = LIBRARY) -> bool:
    if not os.path.exists(library):
        return True
    built = os.path.getmtime(library)
    return any(os.path.getmtime(os.path.join(HERE, f)) > built for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    for library, extra in ((LIBRARY, []), (CHECKED_LIBRARY, ["-DGD_CHECKED"])):
        if force or is_stale(library):
            cmd = ["nvcc", *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), "-o", library,
                   *[os.path.join(HERE, s) for s in SOURCES]]
            subprocess.check_call(cmd, cwd=HERE)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=True))
