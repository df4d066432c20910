"""Build recipe for ``oracle/_ref/libmetal_ref.so`` (TEST INFRASTRUCTURE ONLY).

Takes the reference's Metal kernel bodies from where they lie in a reference checkout
(``mlx-impl/model.py``, the string ``_fused_log_softmax_source``; ``mlx-impl/paged_kv.py``, the
gather kernel's f-string), writes them to scratch files under ``oracle/_ref/`` and compiles ``oracle/metal_emulation.cpp`` around it with g++.  Nothing
of the reference is stored in this repository: ``oracle/_ref/`` is git-ignored, and the scratch
copies of the bodies are deleted once the library is linked.

    python oracle/build_ref.py [path/to/reference]

Without an argument the checkout is looked for in $TOME_REFERENCE, then in a directory named
``reference`` beside this repository.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libmetal_ref.so")


def extract_body(reference_root: str) -> str:
    path = os.path.join(reference_root, "mlx-impl", "model.py")
    with open(path, "r", encoding="utf-8") as fh:
        text = fh.read()
    m = re.search(r'_fused_log_softmax_source\s*=\s*"""(.*?)"""', text, re.S)
    if m is None:
        raise RuntimeError(f"no _fused_log_softmax_source string in {path}")
    return m.group(1)


def extract_gather_body(reference_root: str) -> str:
    """The paged-KV gather body (mlx-impl/paged_kv.py:57-116) is a Python f-string: its fields
    become the emulation's parameter names, its doubled braces single ones."""
    path = os.path.join(reference_root, "mlx-impl", "paged_kv.py")
    with open(path, "r", encoding="utf-8") as fh:
        text = fh.read()
    m = re.search(r'src\s*=\s*f"""(.*?)"""', text, re.S)
    if m is None:
        raise RuntimeError(f"no gather kernel source in {path}")
    body = m.group(1)
    for field in ("B", "H", "D", "block_size", "max_blocks"):
        body = body.replace("{" + field + "}", field + "_arg")
    return body.replace("{{", "{").replace("}}", "}")


def build(reference_root: str | None = None) -> str | None:
    """Returns the library path, or None when no reference checkout is available."""
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    root = reference_root or os.environ.get("TOME_REFERENCE", beside)
    if not os.path.isdir(os.path.join(root, "mlx-impl")):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    body = os.path.join(OUT_DIR, "fused_log_softmax_body.inc")
    gather = os.path.join(OUT_DIR, "gather_paged_kv_body.inc")
    with open(body, "w", encoding="utf-8") as fh:
        fh.write(extract_body(root))
    with open(gather, "w", encoding="utf-8") as fh:
        fh.write(extract_gather_body(root))
    try:
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", OUT_DIR,
               os.path.join(HERE, "metal_emulation.cpp"), "-o", LIB_PATH + ".tmp"]
        subprocess.run(cmd, check=True)
        os.replace(LIB_PATH + ".tmp", LIB_PATH)
    finally:
        os.remove(body)
        os.remove(gather)
    return LIB_PATH


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
