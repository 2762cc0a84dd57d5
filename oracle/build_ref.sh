#!/usr/bin/env bash
# Build the UNMODIFIED reference x86 backend into oracle/_ref/libFastKron.so.
#
# Test infrastructure only: the resulting library is the parity checker and the
# timed CPU baseline.  Nothing in the product path loads it.
#
# The reference generates its kernel translation units into its own source tree
# (src/gen_tuner_kernels.py writes next to itself), so the sources are copied to a
# scratch directory first; only the final shared object lands in oracle/_ref/.
# The generator command is the one the reference's CMakeLists.txt:187 runs for
# ENABLE_X86; the compile flags follow CMakeLists.txt (C++17, -O3, OpenMP, and a
# baseline -march=x86-64-v2: every kernel TU raises its own ISA level with a
# "#pragma GCC target", src/config.h:25-31).
#
# usage: oracle/build_ref.sh <reference_dir> [jobs]   (or FASTKRON_REFERENCE_DIR)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${FASTKRON_REFERENCE_DIR:-}}"
[ -n "$REF" ] || { echo "usage: $0 <reference_dir> (or set FASTKRON_REFERENCE_DIR)" >&2; exit 2; }
JOBS="${2:-$(nproc)}"
OUT="$HERE/_ref"
WORK="${FASTKRON_REF_BUILD_DIR:-${TMPDIR:-/tmp}/fastkron_ref_build}"

if [ ! -f "$REF/include/fastkron.h" ]; then
  echo "reference tree not found at $REF" >&2; exit 2
fi
mkdir -p "$OUT" "$WORK/obj"
rm -rf "$WORK/src" "$WORK/include"
cp -r "$REF/src" "$WORK/src"
cp -r "$REF/include" "$WORK/include"
chmod -R u+w "$WORK"
cd "$WORK"

python3 src/gen_tuner_kernels.py -backend x86 -archs sisd avx avx512 -mm-type mkm kmm \
  -same-factors 2 128,128 -same-factors 2 64,64 -same-factors 3 32,32 \
  -same-factors 5 16,16 -same-factors 7 8,8 -same-factors 10 4,4 -same-factors 20 2,2 \
  -opX N T -opF N T -types float double -batch-type strided \
  -match-configs-file src/kernels/best-kernels/x86-avx-kernels src/kernels/best-kernels/kmm-x86-avx-kernels \
  > "$WORK/gen.log" 2>&1

CXX="g++ -std=c++17 -O3 -march=x86-64-v2 -fopenmp -fPIC -DENABLE_X86 -DFASTKRON_VERSION=1.1.0 -Isrc -Iinclude -w"
for s in fastkron env/env autotuner/autotuner handle/handle handle/distrib_handle \
         kernel_db/kernel_db kernel_db/cpu_kernel_db kmm/kmmalgo kmm/matrix kernels/kmmkernel; do
  echo "src/$s.cpp"
done > "$WORK/core.list"
ls src/kernels/cpu/x86/kron-kernels/*.cpp >> "$WORK/core.list"
export CXX
xargs -a "$WORK/core.list" -P "$JOBS" -I{} sh -c \
  'o=obj/$(echo {} | tr "/" "_" | sed "s/\.cpp$/.o/"); [ -f "$o" ] && [ "$o" -nt {} ] || $CXX -c {} -o "$o"'
g++ -shared -fopenmp -o "$OUT/libFastKron.so" obj/*.o
echo "built $OUT/libFastKron.so ($(ls obj | wc -l) objects)"
