"""Export a trained module to one ``.mim`` file and run it back through the graph runtime.

The file carries weights, metadata and the traced graph; ``mim.open(path).run({...})`` needs no
model code.  The second half builds a graph by hand with ``graph.Builder``: a session with a
variable (a running state that every call updates), the shape of a decoder's key-value cache.
Reference: ``mim.Export`` / ``Model.Run`` / ``Session`` (io/mim/export.go, session.go).
"""
import os
import tempfile

import torch

from mimir_b200 import nn
from mimir_b200 import tensor as T
from mimir_b200.io import export, graph, mim


def main(log=print):
    nn.manual_seed(0)
    net = nn.Sequential(nn.Linear(8, 32), nn.GELU(), nn.LayerNorm(32), nn.Linear(32, 3), nn.Softmax())
    x = T.tensor(torch.randn(4, 8))
    path = os.path.join(tempfile.mkdtemp(), "classifier.mim")
    export.export(path, net, x, input_name="features", output_name="probabilities",
                  dynamic={"features": {0: ("batch", 1024)}}, metadata={"general.name": "demo-classifier"})
    with mim.open(path) as model:
        log("inputs ", model.inputs)
        log("outputs", model.outputs)
        big = T.tensor(torch.randn(100, 8))                 # the batch axis is symbolic
        got = model.run({"features": big})["probabilities"].data()
        err = (got - net(big).data()).abs().max().item()
        log(f"run from file vs module: max difference {err:.2e}")

    # a graph built by hand, with state: an exponential moving average of its input
    b = graph.Builder()
    sample = b.input("sample", "f32", [3])
    state = b.variable("average", "f32", [3])
    new = b.add(b.mul(state, 0.9), b.mul(sample, 0.1))
    b.update(state, new)
    b.output("average", new)
    session = mim.parse(b.serialize()).new_session()
    for _ in range(3):
        avg = session.run({"sample": torch.ones(3)})["average"].data()
    log("moving average after 3 runs:", [round(v, 4) for v in avg.tolist()])
    return err, avg


if __name__ == "__main__":
    main()
