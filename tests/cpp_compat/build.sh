#!/bin/sh
# Builds the reference's OWN gtest suite and basic example, unchanged, against this library's drop-in header
# (include/flash_attn/flash_api.cuh) and the small gtest stand-in beside this script.
# Needs the reference checkout (environment variable REF); outputs go to tests/cpp_compat/_build/ (git-ignored).
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
REF="${REF:-$(cd "$ROOT/.." && pwd)/reference}"  # default: a directory named reference beside this repository
OUT="$HERE/_build"
mkdir -p "$OUT"
FLAGS="-std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -I$ROOT/include -I$HERE -I$REF/tests/cpp"
LINK="-L$ROOT/tinyfa_b200 -ltinyfa_b200 -Xlinker -rpath -Xlinker \$ORIGIN/../../../tinyfa_b200"
nvcc $FLAGS -o "$OUT/ref_suite" "$REF/tests/cpp/test.cpp" "$REF/tests/cpp/test_flash_attn.cu" $LINK
nvcc $FLAGS -o "$OUT/basic_example" "$REF/examples/basic/main.cu" $LINK
echo "built $OUT/ref_suite $OUT/basic_example"
