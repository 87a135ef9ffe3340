#!/bin/sh
# clang-format over the native sources (style: .clang-format)
find torch_dist_ext_b200/csrc tests/cpp baseline/shim -name '*.cu' -o -name '*.cuh' -o -name '*.cpp' -o -name '*.h' | xargs clang-format -i
