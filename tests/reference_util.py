"""Locates an importable copy of the reference package for the tests that exercise its own
find_impl / verify / verify_parity: ``baseline/_ref`` (installed by baseline/install_reference.sh;
travels to the GPU box) or, where the environment variable ``XKERNELS_REFERENCE_SRC`` points at the
``src`` directory of a reference checkout, that source tree."""

import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def reference_available(allow_source_tree: bool) -> bool:
    try:
        import xkernels  # noqa: F401
        return True
    except Exception:
        pass
    candidates = [ROOT / "baseline" / "_ref"]
    if allow_source_tree and os.environ.get("XKERNELS_REFERENCE_SRC"):
        candidates.append(Path(os.environ["XKERNELS_REFERENCE_SRC"]))
    for c in candidates:
        if (c / "xkernels" / "__init__.py").exists():
            sys.path.insert(0, str(c))
            try:
                import xkernels  # noqa: F401
                return True
            except Exception:
                sys.path.remove(str(c))
    return False
