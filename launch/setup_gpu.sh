#!/usr/bin/env bash
# Build the CUDA / C++ extensions in-tree for sm_100a (needs nvcc 12.8+ and the PyTorch of the environment).
set -euo pipefail
cd "$(dirname "$0")/.."
python -m mintext_b200.ops.build
python -c "import mintext_b200; print('mintext_b200', mintext_b200.__version__, 'ready')"
