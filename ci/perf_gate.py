#!/usr/bin/env python
"""Performance gates, the counterpart of the reference's CI gates (ci/cuda/m6.sh:2-17: time no more
than 1.25 x PyTorch on the same GPU; ci/cuda/shard.sh:21-72: 8-GPU efficiency at least 0.85).

    python ci/perf_gate.py ours.json baseline.json [scale_1.json scale_8.json]

``ours.json`` / ``baseline.json`` are the one-line outputs of ``bench.py`` and ``bench.py --impl
baseline`` on the same box; the optional pair are ``bench.py --gpus 1`` and ``--gpus 8`` of the same
build.  Exits 1 when a gate fails."""
import json
import sys

MAX_TIME_RATIO = 1.25      # our step time / PyTorch's
MIN_EFFICIENCY = 0.85      # tokens/s at N GPUs / (N x tokens/s at 1 GPU)


def _load(path):
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                return json.loads(line)
    raise SystemExit(f"{path}: no JSON line")


def main(argv):
    if len(argv) not in (3, 5):
        raise SystemExit(__doc__)
    ours, base = _load(argv[1]), _load(argv[2])
    ok = True
    ratio = ours["ms_per_step"] / base["ms_per_step"]
    print(f"step time: ours {ours['ms_per_step']:.2f} ms, PyTorch {base['ms_per_step']:.2f} ms, ratio {ratio:.3f} "
          f"(gate {MAX_TIME_RATIO})")
    ok &= ratio <= MAX_TIME_RATIO
    if len(argv) == 5:
        one, many = _load(argv[3]), _load(argv[4])
        eff = many["value"] / (many["n_gpus"] * one["value"])
        print(f"scaling: {many['n_gpus']} GPUs at {eff:.3f} of linear (gate {MIN_EFFICIENCY})")
        ok &= eff >= MIN_EFFICIENCY
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv))
