#!/bin/sh
# Puts the UNMODIFIED reference package where the GPU-side fixture generator
# (make_reference_gpu_golden.py, same directory) can import it: the git-ignored baseline/_ref/,
# which travels with the working tree but never enters the history.
#
#   sh tests/golden/install_reference.sh /path/to/vexact-checkout      (or VEXACT_REFERENCE=... in the environment)
#
# First choice is a regular offline pip install.  The project's build backend (hatchling) is not
# in the offline wheelhouse, so that fails here; a wheel of this pure-Python project is nothing
# but its `vexact/` package directory (pyproject.toml: [tool.hatch.build.targets.wheel]
# packages = ["vexact"]), and unpacking that directory into the target is what pip would have done.
# Test infrastructure only: nothing under vexact_b200/ and no timed region of bench.py imports it.
set -e
REF="${1:-${VEXACT_REFERENCE:?give the path of the reference checkout}}"
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
DEST="$ROOT/baseline/_ref"
mkdir -p "$DEST"
if python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
      --target "$DEST" "$REF" >"$DEST/pip_install.log" 2>&1; then
  echo "pip install into $DEST succeeded"
else
  echo "pip install failed ($(tail -n 1 "$DEST/pip_install.log")); unpacking the package directory instead"
  test -d "$DEST/vexact" || cp -r "$REF/vexact" "$DEST/vexact"
fi
python - <<PY
import sys
sys.path.insert(0, "$DEST")
import importlib.util
assert importlib.util.find_spec("vexact") is not None
print("reference importable from $DEST")
PY
