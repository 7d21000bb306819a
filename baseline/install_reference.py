"""Place the reference's BSA path under ``baseline/_ref/`` so that it can run on a GPU machine as the comparator.

    python baseline/install_reference.py [path to a LongCat-Video checkout]

The reference project has no build metadata (no setup.py / pyproject.toml), so it cannot be pip-installed; the two
packages its block-sparse attention needs -- ``longcat_video/block_sparse_attention`` (Triton kernels and their
launchers) and ``longcat_video/context_parallel`` -- and the files of ``longcat_video/modules`` that define one DiT block
are copied unmodified.  ``baseline/_ref/`` is ignored by git:
nothing of the reference enters this repository's history, and nothing in ``longcat_video_b200/`` imports it.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PACKAGES = ["block_sparse_attention", "context_parallel"]
# the DiT block and what it is made of, for the denoising-step harness (bench_dit_step.py); the VAE, the scheduler, the
# avatar model and the quantisation helpers stay behind
MODULE_FILES = ["__init__.py", "attention.py", "blocks.py", "rope_3d.py", "longcat_video_dit.py", "lora_utils.py"]


def install(src_root: str) -> str:
    src_pkg = os.path.join(src_root, "longcat_video")
    if not os.path.isdir(src_pkg):
        raise SystemExit(f"{src_pkg} not found")
    dst_pkg = os.path.join(DEST, "longcat_video")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(dst_pkg)
    open(os.path.join(dst_pkg, "__init__.py"), "w").close()
    for name in PACKAGES:
        shutil.copytree(os.path.join(src_pkg, name), os.path.join(dst_pkg, name), ignore=shutil.ignore_patterns("__pycache__"))
        init = os.path.join(dst_pkg, name, "__init__.py")
        if not os.path.exists(init):
            open(init, "w").close()
    os.makedirs(os.path.join(dst_pkg, "modules"))
    for name in MODULE_FILES:
        src = os.path.join(src_pkg, "modules", name)
        if os.path.exists(src):
            shutil.copy(src, os.path.join(dst_pkg, "modules", name))
    if not os.path.exists(os.path.join(dst_pkg, "modules", "__init__.py")):
        open(os.path.join(dst_pkg, "modules", "__init__.py"), "w").close()
    return DEST


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LONGCAT_VIDEO_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))))
