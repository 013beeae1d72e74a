#!/bin/bash
# Builds the reference's own CPU extension (-DNO_CUDA) in a scratch directory so that
# make_golden.py can import the reference and record golden vectors.  Nothing from the
# reference is copied into this repository: the copy, the generated sources and the built
# module all live under $SCRATCH (default /tmp/spiky_ref).
#
#   usage: tests/golden/build_reference_cpu.sh <reference_checkout> [scratch_dir]
#
# Notes: the reference generates its kernel sources from .proto files by hand (its setup.py
# only does so when run as __main__, after setup()), and the image's default /opt/gcc links
# libstdc++ statically, which breaks the module's iostream use - hence /usr/bin/g++.
set -euo pipefail
REF=${1:?usage: build_reference_cpu.sh <reference_checkout> [scratch_dir]}
SCRATCH=${2:-/tmp/spiky_ref}
mkdir -p "$SCRATCH"
cp -r "$REF/spiky_cuda" "$REF/src" "$SCRATCH/"
cd "$SCRATCH/spiky_cuda"
python - <<'PY'
import contextlib, io
from kernels_logic_parser import generate_cu_from_proto as gen
pairs = [
    ('connections_manager/connections_manager_kernels_logic.proto', 'connections_manager/aux/connections_manager_kernels_logic.cu'),
    ('spnet/spnet_runtime_kernels_logic.proto', 'spnet/aux/spnet_runtime_kernels_logic.cu'),
    ('lut/lut_runtime_kernels_logic.proto', 'lut/aux/lut_runtime_kernels_logic.cu'),
    ('lut/lut_compile_time_kernels_logic.proto', 'lut/aux/lut_compile_time_kernels_logic.cu'),
    ('synapse_growth/synapse_growth_kernels_logic.proto', 'synapse_growth/aux/synapse_growth_kernels_logic.cu'),
    ('misc/spike_storage_kernels_logic.proto', 'misc/aux/spike_storage_kernels_logic.cu'),
    ('torch_utils/torch_utils_kernels_logic.proto', 'torch_utils/aux/torch_utils_kernels_logic.cu'),
]
for src, dst in pairs:
    with contextlib.redirect_stdout(io.StringIO()):
        gen(src, dst)
PY
CC=/usr/bin/gcc CXX=/usr/bin/g++ CFLAGS=-g0 MAX_JOBS=8 python setup.py build_ext --inplace
echo "reference CPU module built; use PYTHONPATH=$SCRATCH/spiky_cuda:$SCRATCH/src"
