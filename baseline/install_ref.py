"""Install the unmodified reference project under baseline/_ref (git-ignored; it travels to the GPU box).

    python baseline/install_ref.py [/path/to/reference]

The reference is a source tree without packaging metadata (no pyproject.toml / setup.py), so
`pip install --target baseline/_ref <tree>` has nothing to build; this recipe first tries pip and, when pip
refuses the tree, installs it the way a pure-Python project is installed: the package directory `qwen3mk/`,
the kernel source `csrc/` it compiles with NVRTC at run time, and `run.py`, byte for byte.  Nothing of the
reference is copied into tracked files.  The result is used only as a measured comparator: the reference's
own kernel through its own `Megakernel` and `bench.steady / isolated` (baseline/time_ref_kernel.py)."""
from __future__ import annotations

import filecmp
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
PARTS = ("qwen3mk", "csrc", "run.py", "requirements.txt")


def install(src: Path = Path("/root/reference")) -> str:
    """Returns a one-line description of what was done ("absent", "pip", "copied", "current")."""
    if not src.is_dir():
        return "absent"
    if all((DEST / p).exists() for p in PARTS) and not filecmp.dircmp(src / "qwen3mk", DEST / "qwen3mk", ignore=["__pycache__"]).diff_files \
            and filecmp.cmp(src / "csrc" / "qwen3_step.cu", DEST / "csrc" / "qwen3_step.cu", shallow=False):
        return "current"
    DEST.mkdir(parents=True, exist_ok=True)
    if (src / "pyproject.toml").exists() or (src / "setup.py").exists():
        r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                            "--find-links", "/opt/wheelhouse", "--target", str(DEST), str(src)], capture_output=True, text=True)
        if r.returncode == 0:
            return "pip"
    for p in PARTS:
        s, d = src / p, DEST / p
        if s.is_dir():
            if d.exists():
                shutil.rmtree(d)
            shutil.copytree(s, d, ignore=shutil.ignore_patterns("__pycache__"))
        elif s.exists():
            shutil.copy2(s, d)
    for f in DEST.rglob("*"):
        if f.is_file():
            f.chmod(0o644)
    return "copied"


if __name__ == "__main__":
    print(install(Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference")))
