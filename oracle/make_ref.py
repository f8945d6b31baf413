"""Place the reference's own Python model beside the oracle, for timing it on the GPU box's host cores.

    python oracle/make_ref.py /path/to/reference/aegist-fast-35b

TEST / MEASUREMENT INFRASTRUCTURE. The reference's CPU implementation of the decode path is its Python
package `aegist` (hybrid.py and the modules it imports). This recipe copies those few files, unmodified,
from the reference tree into `oracle/_ref/aegist/`, which `.gitignore` lists: they are never committed,
they only travel with the working tree to the machine that runs `bench.py`, whose `cpu_baseline` leg and
`--impl reference` arm then time the reference's `HybridLM` itself (kind "reference") instead of the numpy
port (kind "port"). Nothing in the product imports from there. Without an argument, or when the tree is
absent, nothing is done and the port remains the baseline.
"""
import os
import shutil
import sys

FILES = ["__init__.py", "hybrid.py", "model.py", "nx.py", "hc.py", "tokenizer.py"]
HERE = os.path.dirname(os.path.abspath(__file__))


def make_ref(reference_root: str) -> bool:
    src = os.path.join(reference_root, "aegist")
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        return False
    dst = os.path.join(HERE, "_ref", "aegist")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    return True


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print("oracle/_ref ready" if make_ref(sys.argv[1]) else "reference tree not found: nothing done")
