"""Puts a runnable copy of the reference package under oracle/_ref/ (test infrastructure only).

    python oracle/make_ref.py [<reference checkout>]

The reference (bhengubv/shard) is a pure-Python package; "building" it is copying its
`src/shard/*.py` into `oracle/_ref/shard/` unchanged, the equivalent of
`pip install --target oracle/_ref <checkout>` without the metadata.  `oracle/_ref/` is
git-ignored: the copy never enters this repository's history, it only travels with the
working tree (like the built .so files) so that `bench.py --impl reference` can time the
reference's own code on a machine that has no checkout of it.  Nothing in the product
imports it; the only users are `bench.py`'s reference arm and tests that compare against
the reference when it is present.

Exit status 0 with a message when the checkout is absent (nothing to do).
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "shard")
DEFAULT_CHECKOUT = os.environ.get("SHARD_REFERENCE", "/root/reference")


def make_ref(checkout: str = DEFAULT_CHECKOUT, verbose: bool = True) -> str | None:
    """Copy <checkout>/src/shard/*.py to oracle/_ref/shard/; returns the destination or None."""
    src = os.path.join(checkout, "src", "shard")
    if not os.path.isdir(src):
        if verbose:
            print(f"make_ref: no reference checkout at {checkout}; keeping whatever oracle/_ref holds")
        return None
    os.makedirs(DEST, exist_ok=True)
    names = sorted(n for n in os.listdir(src) if n.endswith(".py"))
    for n in names:
        shutil.copyfile(os.path.join(src, n), os.path.join(DEST, n))
    with open(os.path.join(HERE, "_ref", "SOURCE.txt"), "w") as f:
        f.write(f"copied unchanged from {src}: {', '.join(names)}\n")
    if verbose:
        print(f"make_ref: {len(names)} files -> {DEST}")
    return DEST


def ref_path() -> str | None:
    """Directory to put on sys.path to `import shard` (the reference), or None if absent."""
    root = os.path.join(HERE, "_ref")
    return root if os.path.exists(os.path.join(root, "shard", "__init__.py")) else None


if __name__ == "__main__":
    make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
