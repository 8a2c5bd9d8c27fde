"""Recipe that makes the reference package importable as TEST INFRASTRUCTURE.

    python oracle/build_ref.py [/path/to/reference]

Mirrors the reference's own ``lean_transformer`` package, unmodified and from where its checkout lies, into
``oracle/_ref/`` (git-ignored: it never enters this repository's history) and writes a two-class stand-in for the
one dependency that is not installed (``revlib``, imported by ``lean_transformer/sequence.py`` for reversible
layers, which the LeanFFN path never runs).  ``oracle/ref_harness.py`` then imports the mirror with the
monkey-patches newer ``transformers`` releases need.  Only tests, ``__graft_entry__.smoke()`` and the
CPU-baseline legs of ``bench.py`` may use it; the product package never imports anything from here.

Without a reference checkout the script changes nothing and reports that (a machine that only has the mirror
keeps using it).
"""
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
DEFAULT_SOURCE = Path("/root/reference")

REVLIB_STUB = '''"""Stand-in for revlib (not installed): the two names lean_transformer/sequence.py imports.  Reversible layers are
outside the LeanFFN path and are never run through this stand-in."""
import torch.nn as nn


class ReversibleModule(nn.Module):
    pass


class ReversibleSequential(nn.Sequential):
    pass
'''


def build_ref(source: Path = DEFAULT_SOURCE, verbose: bool = True) -> bool:
    """Returns True if ``oracle/_ref`` holds the reference package afterwards."""
    package = Path(source) / "lean_transformer"
    if not package.is_dir():
        if verbose:
            print(f"oracle/_ref: no reference checkout at {source}; "
                  f"{'keeping the existing mirror' if (TARGET / 'lean_transformer').is_dir() else 'nothing to mirror'}")
        return (TARGET / "lean_transformer").is_dir()
    TARGET.mkdir(exist_ok=True)
    destination = TARGET / "lean_transformer"
    if destination.exists():
        shutil.rmtree(destination)
    shutil.copytree(package, destination, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    (TARGET / "revlib.py").write_text(REVLIB_STUB)
    if verbose:
        print(f"oracle/_ref: mirrored {package} -> {destination}")
    return True


if __name__ == "__main__":
    ok = build_ref(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_SOURCE)
    sys.exit(0 if ok else 1)
