#!/usr/bin/env bash
# Build the reference CPU codec (fpgasystems/gcow sw/src/*.c, unmodified) plus a
# thin C-ABI shim into baseline/_ref/libgcowref.so. The reference ships no
# installable Python package, so this is its offline "install". The training scripts under
# hw/models are copied unchanged next to the library.
#   usage: baseline/build_ref.sh [path-to-reference-checkout]
# Without an argument: $GCOW_REFERENCE, else a checkout named "reference" beside this repository.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-${GCOW_REFERENCE:-$here/../../reference}}"
out="$here/_ref"
mkdir -p "$out"
g++ -std=c++11 -O2 -fPIC -shared -w -x c++ \
    -I"$ref/sw/include" \
    "$ref/sw/src/common.c" "$ref/sw/src/stream.c" "$ref/sw/src/encode.c" \
    "$ref/sw/src/decode.c" "$ref/sw/src/zfp.c" "$here/ref_driver.cpp" \
    -o "$out/libgcowref.so"
# the reference's training scripts, byte for byte; bench.py --impl reference imports them from here
mkdir -p "$out/models"
cp "$ref"/hw/models/*.py "$out/models/"
echo "built $out/libgcowref.so and copied hw/models/*.py to $out/models"
