"""Recipe that places the reference project's own hot-path files under ``oracle/_ref/``.

    python oracle/make_ref.py [/path/to/reference]

(default: the ARCB_REFERENCE_ROOT environment variable, else a checkout named ``reference`` next to
this repository).

Copies, unmodified, ``src/{data,transformer,inference,voting}.py`` and
``tests/test_{data,transformer,inference,voting}.py`` from a checkout of the reference project.
``oracle/_ref/`` is listed in .gitignore: the copies are never committed, they are a local build
product like a compiled object, used only as

  * the acceptance suite: ``tests/test_reference_suite.py`` runs those test files unmodified with
    ``src.voting`` / ``src.data`` / ``src.inference`` aliased to this repository's drop-in modules;
  * the timed CPU baseline of ``bench.py`` (``--impl reference`` and ``cpu_baseline``), which calls
    the reference's own ``generate_output`` on the host cores.

Test infrastructure only: nothing under ``mdlarc_scale_b200/`` reads ``oracle/_ref``.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def default_reference_root() -> Path:
    env = os.environ.get("ARCB_REFERENCE_ROOT")
    return Path(env) if env else HERE.parent.parent / "reference"


SRC_FILES = ["data.py", "transformer.py", "inference.py", "voting.py"]
TEST_FILES = ["test_data.py", "test_transformer.py", "test_inference.py", "test_voting.py"]


def available() -> bool:
    return all((DEST / "src" / f).exists() for f in SRC_FILES) and all((DEST / "tests" / f).exists() for f in TEST_FILES)


def make(reference_root: str | Path | None = None, force: bool = False) -> bool:
    """Copy the files; returns False (and leaves ``_ref`` as it is) when the checkout is absent."""
    root = Path(reference_root) if reference_root is not None else default_reference_root()
    if not (root / "src" / "inference.py").exists():
        return False
    if available() and not force:
        return True
    for sub, names in (("src", SRC_FILES), ("tests", TEST_FILES)):
        (DEST / sub).mkdir(parents=True, exist_ok=True)
        for name in names:
            shutil.copyfile(root / sub / name, DEST / sub / name)
    (DEST / "src" / "__init__.py").write_text("")
    return True


def load_reference_modules(prefix: str = "arcref"):
    """Import the copied reference modules as ``<prefix>.data`` / ``.transformer`` / ``.inference`` /
    ``.voting`` (a private package name, so they cannot shadow or be shadowed by anything called
    ``src``).  The reference's intra-package imports (``from src.data import ...`` or relative) are
    satisfied by also registering the package as ``src`` for the duration of the import only."""
    import importlib.util
    import types
    if not available():
        raise RuntimeError("oracle/_ref is empty: run `python oracle/make_ref.py /path/to/reference`")
    pkg = types.ModuleType(prefix)
    pkg.__path__ = [str(DEST / "src")]
    saved = {k: sys.modules.get(k) for k in ("src", "src.data", "src.transformer", "src.inference", "src.voting")}
    sys.modules[prefix] = pkg
    sys.modules["src"] = pkg
    out = {}
    try:
        for name in ("data", "transformer", "voting", "inference"):
            spec = importlib.util.spec_from_file_location(f"{prefix}.{name}", DEST / "src" / f"{name}.py")
            mod = importlib.util.module_from_spec(spec)
            sys.modules[f"{prefix}.{name}"] = mod
            sys.modules[f"src.{name}"] = mod
            spec.loader.exec_module(mod)
            setattr(pkg, name, mod)
            out[name] = mod
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return out


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    ok = make(args[0] if args else None, force="--force" in sys.argv)
    print(f"{DEST}: {'ready' if ok else 'reference checkout not found, nothing copied'}")
    sys.exit(0 if ok else 1)
