#!/usr/bin/env bash
# Rebind check of the reference's Python package: installs the UNMODIFIED reference
# pyfastkron (its .py files and its pybind11 shim pyfastkron/pywrapper.cpp, compiled as is)
# under oracle/_ref/pyfastkron/, with
#   FastKronCUDA  linked against this repository's fastkron_b200/libFastKron.so, and
#   FastKronX86   linked against the reference's own x86 build oracle/_ref/libFastKron.so
# (pyfastkron/fastkronbase.py:9-25 wants both importable).
#
# Test infrastructure only; everything lands in oracle/_ref/ (git-ignored build output).
#
# usage: oracle/build_pyref.sh <reference_dir>   (or FASTKRON_REFERENCE_DIR)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(dirname "$HERE")"
REF="${1:-${FASTKRON_REFERENCE_DIR:-}}"
[ -n "$REF" ] || { echo "usage: $0 <reference_dir> (or set FASTKRON_REFERENCE_DIR)" >&2; exit 2; }
OUT="$HERE/_ref"
[ -f "$REF/pyfastkron/pywrapper.cpp" ] || { echo "reference tree not found at $REF" >&2; exit 2; }
[ -f "$OUT/libFastKron.so" ] || { echo "run oracle/build_ref.sh first" >&2; exit 2; }
[ -f "$REPO/fastkron_b200/libFastKron.so" ] || { echo "build fastkron_b200/csrc first" >&2; exit 2; }

PKG="$OUT/pyfastkron"
mkdir -p "$PKG"
cp "$REF"/pyfastkron/*.py "$PKG"/
SUF="$(python3 -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
INC="$(python3 -m pybind11 --includes)"
CUDA_INC="${CUDA_HOME:-/usr/local/cuda}/include"

# the CUDA module: the shim over THIS library (rpath relative to the module)
g++ -O2 -shared -fPIC -std=c++17 $INC -DENABLE_CUDA "$REF/pyfastkron/pywrapper.cpp" \
    -I"$REPO/include" -I"$CUDA_INC" -L"$REPO/fastkron_b200" -lFastKron \
    -Wl,-rpath,'$ORIGIN/../../../fastkron_b200' -o "$PKG/FastKronCUDA$SUF"
# the x86 module: the shim over the reference's own library.  Both libraries are called
# libFastKron.so and the dynamic loader keys loaded objects by name, so the reference's is
# linked under a second name (a symbolic link) to keep the two apart in one process.
ln -sf libFastKron.so "$OUT/libFastKronRefX86.so"
g++ -O2 -shared -fPIC -std=c++17 $INC -DENABLE_X86 "$REF/pyfastkron/pywrapper.cpp" \
    -I"$REF/include" -L"$OUT" -lFastKronRefX86 -Wl,-rpath,'$ORIGIN/..' -o "$PKG/FastKronX86$SUF"
# the reference's own torch test, byte for byte, for tests/test_pyfastkron_rebind_gpu.py
mkdir -p "$OUT/pytests"
cp "$REF/tests/python/test_torch.py" "$OUT/pytests/test_torch.py"
echo "built $PKG"
