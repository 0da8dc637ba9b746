#!/bin/bash
# Builds the reference's CPU simulator (unmodified sources) with this repo's driver into baseline/_ref/.
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-$HERE/../../reference}
mkdir -p "$HERE/_ref"
g++ -O2 -std=c++11 -w -DNOLOG -include cstring -include cstdint -I"$REF/simulation" -I"$REF/simulation/algorithm" -I"$REF/simulation/scheduler" \
    "$HERE/ref_sim_driver.cpp" "$REF"/simulation/algorithm/*.cpp "$REF"/simulation/scheduler/*.cpp -o "$HERE/_ref/ref_sim"
echo "$HERE/_ref/ref_sim"
