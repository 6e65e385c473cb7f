"""Recipe for the reference-Triton arm of the benchmark: put an importable copy of the reference's
`hattention` package under baseline/_ref/ (git-ignored; it is not part of this repository's source).

    python baseline/make_ref.py /path/to/log-linear-attention      # default: $LLATTN_REFERENCE_CHECKOUT

What it does
  * copies the reference's `hattention/` directory verbatim into baseline/_ref/hattention/;
  * replaces the copy's `__init__.py` by an empty one: the original imports the Hugging Face model
    files, which need `mamba_ssm` and `causal_conv1d` (hattention/__init__.py:3-12); the kernels under
    test do not.
Nothing else in the copy is edited.  The API drift between the reference and the installed
flash-linear-attention / Triton versions is bridged at import time by baseline/ref_compat.py, which
is committed and documents each shim.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(src_root: str) -> None:
    src = os.path.join(src_root, "hattention")
    if not os.path.isdir(src):
        raise SystemExit(f"{src} not found")
    dst_root = os.path.join(HERE, "_ref")
    dst = os.path.join(dst_root, "hattention")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(dst_root, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    with open(os.path.join(dst, "__init__.py"), "w") as f:
        f.write("# emptied by baseline/make_ref.py: the original imports model files that need mamba_ssm\n")
    print(f"reference package copied to {dst}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LLATTN_REFERENCE_CHECKOUT", "/root/reference"))
