"""Clips, the mel front end as a lazy layer and the waveform classifier (reference: audio/wav.go,
features.go, classifier.go and their tests)."""
import io
import math

import torch

import mimir_b200.tensor as T
from mimir_b200 import audio, nn, optim


def tone(freq, rate=16000, seconds=1.0, amp=0.5):
    t = torch.arange(int(rate * seconds)) / rate
    return amp * torch.sin(2 * math.pi * freq * t)


def test_clip_round_trip_resample_and_fit():
    c = audio.Clip(tone(1000), 16000)
    buf = io.BytesIO()
    audio.write_clip(buf, c)
    buf.seek(0)
    back = audio.read_clip(buf)
    assert back.rate == 16000 and float((back.samples - c.samples).abs().max()) < 1e-4 and abs(c.seconds() - 1.0) < 1e-9
    for rate in (8000, 22050):
        r = c.resample(rate)
        n = 4096
        peak = torch.fft.rfft(r.samples[1000:1000 + n]).abs().argmax().item() * rate / n
        assert r.samples.numel() == rate and abs(peak - 1000) < 2 * rate / n and 0.45 < float(r.samples[500:-500].abs().max()) < 0.55
    # a tone above the new Nyquist frequency is removed, not folded back
    assert float(audio.Clip(tone(6000), 16000).resample(8000).samples[500:-500].abs().max()) < 0.02
    assert c.fit(10).samples.numel() == 10 and c.fit(20000).samples[16000:].abs().sum() == 0
    assert audio.Mel().frames(16000) == 101 and audio.Mel(rate=8000).resolve().n_fft == 200


def test_front_end_matches_the_fft_and_carries_gradients():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 4000, generator=g) * 0.1
    want = torch.stack([audio.log_mel(v, 16000) for v in x])
    got = audio.spectrogram(T.tensor(x))
    assert got.shape == (2, 26, 40) and torch.allclose(got.data(), want, atol=1e-4)
    assert audio.MelSpectrogram()(T.tensor(x)).shape == (2, 1, 26, 40)
    assert torch.allclose(audio.mfcc_of(got, 13).data(), torch.stack([audio.mfcc(v, 16000) for v in x]), atol=1e-4)
    p = T.Param(x)
    T.sum_(audio.spectrogram(p.value())).backward()
    assert p.grad().data().abs().sum() > 0
    assert isinstance(audio.spectrogram(T.tensor(torch.zeros(1, 100))).err, T.ErrShape)


def test_classifier_tells_tones_apart_and_swaps_heads():
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)

    def batch(n=16):
        y = torch.randint(0, 2, (n,), generator=g)
        freq = torch.where(y == 0, 400.0, 2500.0) * (1 + 0.1 * (torch.rand(n, generator=g) - 0.5))
        x = torch.stack([tone(float(f), seconds=0.2) for f in freq]) + 0.05 * torch.randn(n, 3200, generator=g)
        return x, y
    clf = audio.WaveClassifier(2, width=0.25)
    opt = optim.Adam(clf.parameters(), lr=1e-2)
    for _ in range(25):
        x, y = batch()
        nn.loss.cross_entropy(clf(T.tensor(x)), T.tensor(y)).backward()
        opt.step()
        opt.zero_grad()
    clf.eval()
    x, y = batch(32)
    assert (clf(T.tensor(x)).data().argmax(1) == y).float().mean() > 0.9
    assert clf.features(T.tensor(x)).shape == (32, clf.width)
    clf.set_head(5)
    assert clf(T.tensor(x)).shape == (32, 5) and len(clf.head_parameters()) == 2
