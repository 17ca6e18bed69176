#!/bin/bash
# Installs the UNMODIFIED reference package (pure Python) next to the repository, under baseline/_ref/ (git-ignored; it
# travels to the GPU box with the built libraries).  The reference's build backend (hatchling) is not in the offline
# wheelhouse, so the install runs from a scratch copy whose only change is the [build-system] table of pyproject.toml
# (setuptools instead of hatchling); the package files are installed as they are.
#   usage: baseline/install_reference.sh /path/to/StateQuant
set -e
SRC=${1:?path of the reference checkout}
ROOT=$(cd "$(dirname "$0")/.." && pwd)
TMP=$(mktemp -d)
cp -r "$SRC/src" "$SRC/pyproject.toml" "$SRC/README.md" "$SRC/LICENSE" "$TMP/" 2>/dev/null || cp -r "$SRC/src" "$SRC/pyproject.toml" "$TMP/"
python - "$TMP/pyproject.toml" <<'PY'
import re, sys
p = sys.argv[1]
s = open(p).read()
s = re.sub(r'\[build-system\].*?(?=\n\[project\])', '[build-system]\nrequires = ["setuptools"]\nbuild-backend = "setuptools.build_meta"\n', s, flags=re.S)
s = s.replace('dynamic = ["version"]', 'version = "0.1.1"')
s = re.sub(r'license = "Apache-2.0"\nlicense-files = \["LICENSE"\]\n', '', s)
s = re.sub(r'\[tool\.hatch\.version\].*', '[tool.setuptools.packages.find]\nwhere = ["src"]\n', s, flags=re.S)
open(p, 'w').write(s)
PY
rm -rf "$ROOT/baseline/_ref"
python -m pip install --no-index --no-build-isolation --no-deps --target "$ROOT/baseline/_ref" "$TMP" 2>&1 | tail -2
rm -rf "$TMP"
ls "$ROOT/baseline/_ref"
