#!/bin/bash
# Installs the UNMODIFIED reference package into baseline/_ref (git-ignored) so that the GPU tests
# can run the reference's own find_impl / verify / verify_parity against the cards of this repo.
# The wheel omits the reference's registry/ data directory (JSON specs, cards, sweeps, schemas), so
# it is copied next to the package.  Usage:  baseline/install_reference.sh /path/to/xkernels
set -euo pipefail
REF="${1:?usage: baseline/install_reference.sh /path/to/xkernels}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$REF" "$TMP/src"            # the build writes into the source tree; the original may be read-only
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" --upgrade "$TMP/src"
rm -rf "$HERE/_ref/registry"
cp -r "$REF/registry" "$HERE/_ref/registry"
rm -rf "$TMP"
echo "installed into $HERE/_ref"
