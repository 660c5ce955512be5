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
