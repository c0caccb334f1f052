#!/bin/sh
# Compile the reference's own C graph builder (the Cython-generated cygraph.c,
# which #includes fast_converter_libraries/create_graph.c) straight from the
# reference tree into oracle/_ref/.  Outputs only; no reference source is copied.
# Usage: oracle/build_ref.sh [reference_root]
set -e
REF="${1:-${MATRIS_REFERENCE_ROOT:?set MATRIS_REFERENCE_ROOT or pass the reference root}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
[ -f "$REF/matris/graph/cygraph.c" ] || { echo "reference tree not found under $REF" >&2; exit 3; }
mkdir -p "$HERE/_ref"
PYINC="$(python -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
NPINC="$(python -c 'import numpy; print(numpy.get_include())')"
SUFFIX="$(python -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
gcc -O2 -shared -fPIC -w -I"$PYINC" -I"$NPINC" -I"$REF/matris/graph" \
    "$REF/matris/graph/cygraph.c" -o "$HERE/_ref/cygraph$SUFFIX"
echo "built $HERE/_ref/cygraph$SUFFIX"
