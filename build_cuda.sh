#!/bin/sh
# Builds the native extension and the standalone C++ harness for sm_100a (in-tree), then prints
# where they are. Counterpart of the reference's one-line build_cuda.sh (nvcc ... -arch sm_80).
set -e
cd "$(dirname "$0")"
python -m torch_dist_ext_b200._build "$@"
echo "harness: tests/cpp/unit_test.bin [ranks] [emulate]"
