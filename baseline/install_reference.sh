#!/usr/bin/env bash
# Install the UNMODIFIED reference package (SuriyaaMM/feather) into baseline/_ref/
# so that its own Triton kernels and packer can be run beside this library on a
# GPU box (tests/test_reference_gpu.py, bench.py's reference legs).
#
#   baseline/install_reference.sh /path/to/reference/checkout
#
# The reference's pyproject lists only the top-level package, and its
# sub-packages feather/packers and feather/routines have no __init__.py, so a
# plain `pip install` would leave them out.  The install therefore runs from a
# scratch copy whose package list names the two sub-packages as well; no source
# file of the reference is changed.  baseline/_ref/ is git-ignored: nothing of
# the reference enters this repository's history.
set -euo pipefail
SRC="${1:?usage: install_reference.sh <reference checkout>}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
DST="$HERE/_ref"
TMP="$(mktemp -d /tmp/feather_ref_src.XXXXXX)"
trap 'rm -rf "$TMP"' EXIT
cp -r "$SRC/feather" "$SRC/pyproject.toml" "$SRC/README.md" "$SRC/LICENSE" "$TMP/"
sed -i 's/^packages = \["feather"\]/packages = ["feather", "feather.packers", "feather.routines"]/' "$TMP/pyproject.toml"
rm -rf "$DST"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$DST" "$TMP"
ls "$DST/feather/packers/fp8.py" "$DST/feather/routines/gemv.py" "$DST/feather/routines/dot.py"
