"""Audio front end and classifier (reference: audio/): WAV I/O, STFT, mel filter bank, log-mel,
MFCC, a small convolutional classifier over log-mel frames."""
from __future__ import annotations

import math
import struct

import torch

from .. import nn
from .. import tensor as T


def read_wav(path: str):
    """PCM 8/16/24/32-bit or float32 WAV -> ``(samples float32 [frames, channels] in [-1, 1], rate)``."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        cid, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        body = data[pos + 8:pos + 8 + size]
        if cid == b"fmt ":
            fmt = struct.unpack("<HHIIHH", body[:16])
        elif cid == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError("WAV file without fmt or data chunk")
    tag, ch, rate, _, _, bits = fmt
    if tag == 3 and bits == 32:
        x = torch.frombuffer(bytearray(pcm), dtype=torch.float32).clone()
    elif tag in (1, 0xFFFE) and bits == 16:
        x = torch.frombuffer(bytearray(pcm), dtype=torch.int16).float() / 32768.0
    elif tag in (1, 0xFFFE) and bits == 8:
        x = (torch.frombuffer(bytearray(pcm), dtype=torch.uint8).float() - 128.0) / 128.0
    elif tag in (1, 0xFFFE) and bits == 32:
        x = torch.frombuffer(bytearray(pcm), dtype=torch.int32).float() / 2147483648.0
    elif tag in (1, 0xFFFE) and bits == 24:
        b = torch.frombuffer(bytearray(pcm), dtype=torch.uint8).view(-1, 3).int()
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = torch.where(v >= 1 << 23, v - (1 << 24), v).float() / float(1 << 23)
    else:
        raise ValueError(f"unsupported WAV encoding: tag {tag}, {bits} bits")
    return x.view(-1, ch), rate


def write_wav(path: str, samples: torch.Tensor, rate: int) -> None:
    x = samples if samples.dim() == 2 else samples[:, None]
    pcm = (x.clamp(-1, 1) * 32767.0).round().to(torch.int16).contiguous().numpy().tobytes()
    ch = x.shape[1]
    hdr = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, ch, rate, rate * ch * 2, ch * 2, 16)
    with open(path, "wb") as f:
        f.write(hdr + b"data" + struct.pack("<I", len(pcm)) + pcm)


def hz_to_mel(f):
    return 2595.0 * math.log10(1.0 + f / 700.0)


def mel_to_hz(m):
    return 700.0 * (10.0 ** (m / 2595.0) - 1.0)


def mel_filterbank(n_mels: int, n_fft: int, rate: int, fmin: float = 0.0, fmax: float | None = None) -> torch.Tensor:
    """Triangular filters [n_mels, n_fft // 2 + 1] (HTK mel scale)."""
    fmax = fmax or rate / 2
    mels = torch.linspace(hz_to_mel(fmin), hz_to_mel(fmax), n_mels + 2)
    hz = 700.0 * (10.0 ** (mels / 2595.0) - 1.0)
    freqs = torch.linspace(0, rate / 2, n_fft // 2 + 1)
    lo, mid, hi = hz[:-2, None], hz[1:-1, None], hz[2:, None]
    up, down = (freqs[None] - lo) / (mid - lo), (hi - freqs[None]) / (hi - mid)
    return torch.minimum(up, down).clamp_min(0)


def stft_power(x: torch.Tensor, n_fft: int = 400, hop: int = 160) -> torch.Tensor:
    """x [..., samples] -> power spectrogram [..., frames, n_fft // 2 + 1] (Hann window, centred)."""
    win = torch.hann_window(n_fft, periodic=True, device=x.device)
    s = torch.stft(x, n_fft, hop, window=win, center=True, pad_mode="reflect", return_complex=True)
    return (s.real ** 2 + s.imag ** 2).transpose(-1, -2)


def log_mel(x, rate: int = 16000, n_fft: int = 400, hop: int = 160, n_mels: int = 40, eps: float = 1e-10):
    p = stft_power(x, n_fft, hop)
    return torch.log(p @ mel_filterbank(n_mels, n_fft, rate).to(p).t() + eps)


def dct_matrix(n_out: int, n_in: int) -> torch.Tensor:
    """Orthonormal DCT-II."""
    k = torch.arange(n_out)[:, None].float()
    n = torch.arange(n_in)[None].float()
    m = torch.cos(math.pi / n_in * (n + 0.5) * k) * math.sqrt(2.0 / n_in)
    m[0] /= math.sqrt(2.0)
    return m


def mfcc(x, rate: int = 16000, n_mfcc: int = 13, **kw):
    lm = log_mel(x, rate, **kw)
    return lm @ dct_matrix(n_mfcc, lm.shape[-1]).to(lm).t()


class Classifier(nn.Module):
    """Keyword-spotting sized CNN over log-mel frames [B, 1, frames, mels]."""

    def __init__(self, classes: int, width: int = 32):
        self.body = nn.Sequential(
            nn.Conv2d(1, width, 3, padding=1), nn.BatchNorm2d(width), nn.ReLU(), nn.MaxPool2d(2),
            nn.Conv2d(width, 2 * width, 3, padding=1), nn.BatchNorm2d(2 * width), nn.ReLU(), nn.MaxPool2d(2),
            nn.Conv2d(2 * width, 4 * width, 3, padding=1), nn.BatchNorm2d(4 * width), nn.ReLU())
        self.head = nn.Linear(4 * width, classes)

    def forward(self, x):
        return self.head(T.mean(self.body(x), dim=(2, 3)))


# ---------------------------------------------------------------------------------------------
# Clips, the mel front end as a lazy-tensor layer, and a classifier of waveforms
# (reference: audio/wav.go, audio/features.go, audio/classifier.go)
# ---------------------------------------------------------------------------------------------
from dataclasses import dataclass  # noqa: E402


@dataclass
class Clip:
    """Mono samples in [-1, 1] at ``rate`` samples a second."""

    samples: torch.Tensor
    rate: int

    def seconds(self) -> float:
        return self.samples.numel() / float(max(self.rate, 1))

    def resample(self, rate: int) -> "Clip":
        """The clip at another rate: band-limited (windowed-sinc) interpolation, with the cut-off at the lower
        of the two Nyquist frequencies so that slowing down does not alias."""
        if rate <= 0:
            raise ValueError("resample: the rate must be positive")
        if rate == self.rate or self.samples.numel() == 0:
            return Clip(self.samples.clone(), rate)
        x = self.samples.double()
        n_out = max(1, int(round(x.numel() * rate / self.rate)))
        ratio = self.rate / rate
        cutoff = min(1.0, rate / self.rate)                    # relative to the source's Nyquist frequency
        half = int(math.ceil(16 / cutoff))
        t = torch.arange(n_out, dtype=torch.double) * ratio     # positions in source samples
        base = t.floor().long()
        k = torch.arange(-half + 1, half + 1)
        idx = base[:, None] + k[None]
        d = t[:, None] - idx.double()
        w = cutoff * torch.sinc(cutoff * d) * (0.5 + 0.5 * torch.cos(math.pi * d / half)).clamp_min(0)
        w = torch.where(d.abs() <= half, w, torch.zeros_like(w))
        y = (x[idx.clamp(0, x.numel() - 1)] * w).sum(1)
        return Clip(y.float(), rate)

    def fit(self, n: int) -> "Clip":
        """Exactly ``n`` samples: cut at the end, or padded with silence."""
        s = self.samples[:n]
        return Clip(torch.cat([s, torch.zeros(n - s.numel())]) if s.numel() < n else s.clone(), self.rate)


def read_clip(src) -> Clip:
    """A WAV file (path or binary file object) as a mono clip: channels are averaged."""
    if hasattr(src, "read"):
        import os
        import tempfile
        with tempfile.NamedTemporaryFile(delete=False, suffix=".wav") as f:
            f.write(src.read())
        try:
            x, rate = read_wav(f.name)
        finally:
            os.unlink(f.name)
    else:
        x, rate = read_wav(src)
    return Clip(x.mean(1), rate)


def write_clip(dst, clip: Clip) -> None:
    if hasattr(dst, "write"):
        import os
        import tempfile
        with tempfile.NamedTemporaryFile(delete=False, suffix=".wav") as f:
            name = f.name
        try:
            write_wav(name, clip.samples, clip.rate)
            with open(name, "rb") as f:
                dst.write(f.read())
        finally:
            os.unlink(name)
    else:
        write_wav(dst, clip.samples, clip.rate)


@dataclass
class Mel:
    """The front end's sizes: a zero takes the default (16 kHz, 25 ms windows every 10 ms, 40 bands to Nyquist)."""

    rate: int = 0
    n_fft: int = 0
    hop: int = 0
    mels: int = 0
    fmin: float = 0.0
    fmax: float = 0.0

    def resolve(self) -> "Mel":
        rate = self.rate or 16000
        n_fft = self.n_fft or int(round(0.025 * rate))
        return Mel(rate, n_fft, self.hop or int(round(0.010 * rate)), self.mels or 40, self.fmin, self.fmax or rate / 2)

    def frames(self, n: int) -> int:
        """How many frames ``n`` samples give."""
        return 1 + n // self.resolve().hop


def filterbank(m: Mel) -> torch.Tensor:
    m = m.resolve()
    return mel_filterbank(m.mels, m.n_fft, m.rate, m.fmin, m.fmax)


def _dft(n_fft: int):
    """Windowed real DFT as two matrices ``[n_fft, bins]``: the transform is then a pair of GEMMs."""
    n = torch.arange(n_fft, dtype=torch.double)[:, None]
    k = torch.arange(n_fft // 2 + 1, dtype=torch.double)[None]
    win = torch.hann_window(n_fft, periodic=True, dtype=torch.double)[:, None]
    ang = 2 * math.pi * n * k / n_fft
    return (win * torch.cos(ang)).float(), (win * -torch.sin(ang)).float()


def spectrogram(x, m: Mel = Mel(), eps: float = 1e-10):
    """Log-mel spectrogram of waveforms ``x [batch, samples]`` (a lazy tensor) as ``[batch, frames, mels]``,
    in lazy tensor ops: reflect padding by half a window, overlapping frames as a strided view, the windowed
    DFT as two matrix products, the mel bands as a third.  Gradients flow to ``x``."""
    m = m.resolve()
    if not isinstance(x, T.Tensor):
        x = T.tensor(torch.as_tensor(x, dtype=torch.float32))
    if len(x.shape) == 1:
        x = T.unsqueeze(x, 0)
    b, n = x.shape
    pad = m.n_fft // 2
    if n <= pad:
        return T.core._error_tensor(T.ErrShape(f"spectrogram: {n} samples, a window is {m.n_fft}"))
    left = T.flip(T.shrink(x, ((0, b), (1, pad + 1))), (1,))
    right = T.flip(T.shrink(x, ((0, b), (n - pad - 1, n - 1))), (1,))
    frames = T.windows(T.cat([left, x, right], 1), 1, m.n_fft, m.hop)            # [b, frames, n_fft]
    cos, sin = _dft(m.n_fft)
    dev = x.device
    re, im = T.matmul(frames, T.tensor(cos, device=dev)), T.matmul(frames, T.tensor(sin, device=dev))
    power = re * re + im * im
    return T.log(T.matmul(power, T.tensor(filterbank(m).t().contiguous(), device=dev)) + eps)


class MelSpectrogram(nn.Module):
    """``[batch, samples] -> [batch, 1, frames, mels]`` log-mel pictures: the front end as a layer, so a model
    that starts with it reads waveforms and is exported whole."""

    def __init__(self, m: Mel = Mel()):
        self._nn_skip_cfg = m.resolve()

    def config(self) -> Mel:
        return self._nn_skip_cfg

    def forward(self, x):
        return T.unsqueeze(spectrogram(x, self._nn_skip_cfg), 1)


def mfcc_of(log_mel_frames, n: int = 13):
    """The first ``n`` cepstral coefficients of log-mel frames ``[..., frames, mels]`` (a lazy tensor):
    an orthonormal DCT-II over the bands."""
    d = dct_matrix(n, log_mel_frames.shape[-1]).t().contiguous()
    return T.matmul(log_mel_frames, T.tensor(d, device=log_mel_frames.device))


class WaveClassifier(nn.Module):
    """Waveforms to class logits: the mel front end, three convolution stages over the log-mel picture
    (normalised per clip), the average over time and bands, and a linear head.  ``features`` / ``width`` /
    ``set_head`` / ``head_parameters`` split what it hears from what it says, for transfer learning."""

    def __init__(self, classes: int, mel: MelSpectrogram | None = None, width: float = 1.0):
        self.mel = mel or MelSpectrogram()
        w = max(4, int(round(32 * width)))
        self.body = nn.Sequential(
            nn.Conv2d(1, w, 3, padding=1), nn.BatchNorm2d(w), nn.ReLU(), nn.MaxPool2d(2),
            nn.Conv2d(w, 2 * w, 3, padding=1), nn.BatchNorm2d(2 * w), nn.ReLU(), nn.MaxPool2d(2),
            nn.Conv2d(2 * w, 4 * w, 3, padding=1), nn.BatchNorm2d(4 * w), nn.ReLU())
        self.width = 4 * w
        self.head = nn.Linear(self.width, classes)

    def features(self, x):
        p = self.mel(x)
        mean = T.mean(p, dim=(2, 3), keepdim=True)
        d = p - mean
        p = d / T.sqrt(T.mean(d * d, dim=(2, 3), keepdim=True) + 1e-5)
        return T.mean(self.body(p), dim=(2, 3))

    def forward(self, x):
        return self.head(self.features(x))

    def set_head(self, classes: int) -> None:
        self.head = nn.Linear(self.width, classes)

    def head_parameters(self) -> list:
        return self.head.parameters()
