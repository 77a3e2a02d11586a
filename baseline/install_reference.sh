#!/bin/bash
# Installs the UNMODIFIED reference package (MoonshotAI/MoBA, `moba`) from a local checkout into baseline/_ref
# (git-ignored). No index access, no dependency resolution:
# torch, transformers, einops and flash-attn come from the image.
#   usage: baseline/install_reference.sh [path-to-reference-checkout]     (default: $MOBA_REFERENCE_SRC)
set -e
SRC="${1:-${MOBA_REFERENCE_SRC:-/root/reference}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$SRC" "$TMP/src"          # the build writes egg-info into the source tree; the checkout is read-only
python -m pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --no-deps \
    --target "$HERE/_ref" --upgrade "$TMP/src"
rm -rf "$TMP"
