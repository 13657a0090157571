#!/bin/sh
# Builds sampler_golden.cpp against a checkout of jiamumuzhao/vllm-cpp (first argument) with the
# host compiler only and writes sampler_golden.json beside this script.
set -e
REF="$1"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
g++ -std=c++17 -O1 -I "$REF/include" "$HERE/sampler_golden.cpp" "$REF/src/sampler/sampler.cpp" \
    "$REF/src/sampler/topk_topp.cpp" -o "$TMP/sampler_golden"
"$TMP/sampler_golden" > "$HERE/sampler_golden.json"
rm -r "$TMP"
