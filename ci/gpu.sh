#!/usr/bin/env bash
# GPU tier (one B200 or more): kernel tests against fp32 PyTorch, the conformance table, one smoke step, the headline
# benchmark for both arms, and the perf gate over their JSON lines.  Multi-GPU tests skip below 2 GPUs.
set -euo pipefail
cd "$(dirname "$0")/.."
python -c "import __graft_entry__ as g; g.build()"
python -m pytest tests -x -q -m gpu
python -c "import __graft_entry__ as g; g.smoke()"
N=${N:-1}
mkdir -p ci/out
if [ "$N" -gt 1 ]; then
  RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1 --master-port 29631"
else
  RUN=python
fi
$RUN bench.py --gpus "$N" --steps 20 --warmup 5 | tee ci/out/ours.json
$RUN bench.py --gpus "$N" --steps 20 --warmup 5 --impl baseline | tee ci/out/baseline.json
python ci/perf_gate.py ci/out/ours.json ci/out/baseline.json
