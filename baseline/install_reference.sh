#!/bin/bash
# Installs the unmodified reference sources into baseline/_ref (git-ignored).  The reference ships no
# setup.py / pyproject.toml, so it is installed from a scratch copy that only adds a packaging stub.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC="${1:?usage: install_reference.sh <path of the reference checkout>}"
TMP="$(mktemp -d /tmp/bf_ref_XXXX)"
cp -r "$SRC"/. "$TMP"/
rm -rf "$TMP/.git"
for d in gt_sp models utils; do touch "$TMP/$d/__init__.py"; done
cat > "$TMP/setup.py" <<'PY'
from setuptools import setup
setup(name="budgetformer-reference", version="0.0", packages=["gt_sp", "models", "utils"],
      py_modules=["main_node_fullgraph_sp", "main_node_sp"])
PY
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse --target "$HERE/_ref" "$TMP"
rm -rf "$TMP"
ls "$HERE/_ref"
