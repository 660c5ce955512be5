#!/usr/bin/env bash
# CPU tier: build the native library (nvcc cross-compiles sm_100a without a GPU), then every test that needs no GPU
# (distributed paths run as gloo ranks on 127.0.0.1).
set -euo pipefail
cd "$(dirname "$0")/.."
python -c "import __graft_entry__ as g; g.build()"
python -m pytest tests -x -q -m "not gpu"
# classical models against scikit-learn on this machine, where it is installed: none may take twice its time
if python -c "import sklearn" 2>/dev/null; then
  python -m mimir_b200.utils.bench_ml --rows 20000 --gate 2
fi
