"""The example programs run and learn on the CPU (short settings)."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples"))

quiet = lambda *a, **k: None  # noqa: E731


def test_gpt2_example_learns():
    import gpt2_train
    losses = gpt2_train.cpu_main(steps=25, log=quiet)
    assert sum(losses[-3:]) / 3 < sum(losses[:3]) / 3 - 0.2


def test_llama_generate_example():
    import llama_generate
    out, text = llama_generate.main(prompt="hi", n=5, log=quiet)
    assert len(out) <= 5 and isinstance(text, str)
    assert llama_generate.main(prompt="hi", n=5, log=quiet)[0] == out        # same seed, same sample


def test_mnist_example_learns():
    import mnist
    reports = mnist.main(model="mlp", epochs=3, log=quiet)
    assert reports[-1].loss < reports[0].loss


def test_generative_examples():
    import generative
    v = generative.vae_main(steps=60, log=quiet)
    assert v[-1] < v[0]
    g = generative.gan_main(steps=20, log=quiet)
    assert len(g) == 20 and all(d == d and gl == gl for d, gl in g)          # finite
    h, x = generative.diffusion_main(steps=80, timesteps=20, log=quiet)
    assert sum(h[-10:]) < sum(h[:10]) and x.shape == (256, 2)


def test_gnn_example():
    import gnn
    assert gnn.main(steps=40, log=quiet) > 0.7


def test_export_run_example():
    import export_run
    err, avg = export_run.main(log=quiet)
    assert err < 1e-5
    assert abs(avg[0].item() - (1 - 0.9 ** 3)) < 1e-6


def test_tabular_example():
    import tabular
    a_boost, a_lin, a_auto, agree, err = tabular.main(rows=1500, budget=10.0, log=quiet)
    assert a_boost > 0.85 > a_lin            # the answer is an interaction of two features
    assert a_auto > 0.85 and agree > 0.98 and err < 1e-4
