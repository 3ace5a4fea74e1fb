"""Build recipe for the parity checkers (test infrastructure, not product code).

Two shared objects come out of it:

* ``oracle/libwalk_oracle.so`` -- the C restatement in ``walk_oracle.c`` (gcc).
* ``oracle/_ref/libref_walk.so`` -- the reference's own ``RandomWalk.cpp`` and
  ``BiasedRandomWalk.cpp``, compiled unmodified from where the reference checkout
  lies (``$WALK_REFERENCE_DIR``, else a directory ``reference`` beside this
  repository) against the header stand-ins in ``mlx_stub/`` plus ``ref_harness.cpp``.
  Only built when that checkout is present; the built file is what travels to
  machines that have no checkout. ``python oracle/build.py --require-ref`` fails
  with a message when neither the checkout nor a built library is there.

Run as ``python oracle/build.py``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REFERENCE_DIR = Path(os.environ.get("WALK_REFERENCE_DIR") or HERE.parent.parent / "reference")
ORACLE_SO = HERE / "libwalk_oracle.so"
REF_SO = HERE / "_ref" / "libref_walk.so"


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).exists() and Path(s).stat().st_mtime > t for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "walk_oracle.c"
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off",
               "-o", str(ORACLE_SO), str(src), "-lm"]
        subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_sources():
    return [REFERENCE_DIR / "random_walks" / "RandomWalk.cpp",
            REFERENCE_DIR / "random_walks" / "BiasedRandomWalk.cpp"]


def build_ref(force: bool = False):
    """Compile the reference's two walk sources in place. Returns None when the
    reference checkout is absent and no prebuilt library exists."""
    srcs = reference_sources()
    if not all(s.exists() for s in srcs):
        return REF_SO if REF_SO.exists() else None
    harness = HERE / "ref_harness.cpp"
    stub = HERE / "mlx_stub"
    deps = [harness, *srcs, *stub.rglob("*.h")]
    if force or _stale(REF_SO, deps):
        REF_SO.parent.mkdir(exist_ok=True)
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w",
               f"-I{stub}", f"-I{REFERENCE_DIR}", "-o", str(REF_SO), str(harness), *map(str, srcs)]
        subprocess.run(cmd, check=True)
    return REF_SO


def main() -> int:
    print("oracle:", build_oracle(force="--force" in sys.argv))
    ref = build_ref(force="--force" in sys.argv)
    print("reference build:", ref if ref else "skipped (no reference checkout)")
    if ref is None and "--require-ref" in sys.argv:
        print(f"no reference checkout at {REFERENCE_DIR} (set WALK_REFERENCE_DIR) and no built {REF_SO}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
