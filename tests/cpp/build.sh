#!/bin/sh
# Builds tests/cpp/test_compat against the in-tree libbdattn.so and liboracle.so.
set -e
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
nvcc -std=c++17 -O2 -x cu -I"$ROOT/include" "$ROOT/tests/cpp/test_compat.cpp" \
    -L"$ROOT/brodiffusion_b200" -lbdattn -L"$ROOT/oracle" -loracle \
    -Xlinker -rpath -Xlinker "$ROOT/brodiffusion_b200" -Xlinker -rpath -Xlinker "$ROOT/oracle" \
    -o "$ROOT/tests/cpp/test_compat"
