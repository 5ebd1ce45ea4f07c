"""Writes tests/golden/abi_layout.txt: the layout table of the boundary structs as tests/abi_probe.c
prints it when compiled against the REFERENCE's headers (run where the reference checkout exists:
YVEX_REF names it, default ../reference beside this repository)."""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def reference_table(ref):
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "abi_ref")
        subprocess.run(["gcc", "-std=c11", "-DYVEX_ABI_REF", "-I", os.path.join(ref, "include"), "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "tests", "abi_probe.c"), "-o", exe], check=True)
        return subprocess.run([exe], check=True, capture_output=True, text=True).stdout


if __name__ == "__main__":
    ref = os.environ.get("YVEX_REF") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(ref, "include", "yvex")):
        sys.exit("no reference checkout at " + ref)
    with open(os.path.join(HERE, "abi_layout.txt"), "w") as f:
        f.write(reference_table(ref))
    print("wrote abi_layout.txt")
