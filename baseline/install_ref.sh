#!/usr/bin/env bash
# Installs the unmodified reference packages into baseline/_ref (git-ignored; it travels to the GPU
# box with the working tree).  Needs the reference checkout; run it where that exists:
#     bash baseline/install_ref.sh /path/to/reference
# The two packages are pure Python (setuptools); they are installed from a scratch copy because
# setuptools writes egg-info into the source tree and the checkout may be read-only.  The
# reference's benchmark harness and shape fixtures are not part of its packages; they are copied
# beside them (tools/, fixtures/) so that the harness can be run against this library
# (--candidate-varlen varlenabsorbflashattn_b200:packed_varlen_attn).
set -euo pipefail
REF="${1:?usage: bash baseline/install_ref.sh /path/to/reference-checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
DST="$HERE/_ref"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
mkdir -p "$DST"
for pkg in triton_fa_varlen_v2 triton_target_attn_absorb; do
  cp -r "$REF/$pkg" "$TMP/$pkg"
  python -m pip install --no-index --no-build-isolation --no-deps --upgrade \
      --find-links /opt/wheelhouse --target "$DST" "$TMP/$pkg"
done
mkdir -p "$DST/tools" "$DST/fixtures"
cp "$REF/triton_fa_varlen_v2/tools/benchmark_packed_varlen_flash_attn.py" "$DST/tools/"
cp "$REF/triton_fa_varlen_v2/fixtures/stage1_shapes.jsonl" "$DST/fixtures/"
cp "$REF/triton_target_attn_absorb/fixtures/real_shape_all.json" "$DST/fixtures/"
echo "installed into $DST:"; ls "$DST"
