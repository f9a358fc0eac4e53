"""Signal processing (``crates/torsh-signal``): windows, STFT / ISTFT / spectrogram / mel filterbank, FIR design and
filtering, resampling, Haar wavelet transform."""
from __future__ import annotations

import math

import torch


def window(kind: str, n: int, periodic: bool = True, **kw) -> torch.Tensor:
    f = {"hann": torch.hann_window, "hamming": torch.hamming_window, "blackman": torch.blackman_window,
         "bartlett": torch.bartlett_window}.get(kind)
    if f is not None:
        return f(n, periodic=periodic)
    if kind == "kaiser":
        return torch.kaiser_window(n, periodic=periodic, beta=kw.get("beta", 12.0))
    if kind in ("rect", "boxcar"):
        return torch.ones(n)
    if kind == "gaussian":
        t = torch.arange(n) - (n - 1) / 2
        return torch.exp(-0.5 * (t / kw.get("std", n / 6)) ** 2)
    raise ValueError(f"unknown window {kind!r}")


def stft(x, n_fft=512, hop=None, win="hann", center=True):
    w = window(win, n_fft).to(x)
    return torch.stft(x, n_fft, hop or n_fft // 4, window=w, center=center, return_complex=True)


def istft(X, n_fft=512, hop=None, win="hann", length=None):
    w = window(win, n_fft).to(X.real)
    return torch.istft(X, n_fft, hop or n_fft // 4, window=w, length=length)


def spectrogram(x, n_fft=512, hop=None, power=2.0):
    return stft(x, n_fft, hop).abs() ** power


def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int, fmin=0.0, fmax=None) -> torch.Tensor:
    fmax = fmax or sample_rate / 2
    mel = lambda f: 2595 * math.log10(1 + f / 700)
    inv = lambda m: 700 * (10 ** (m / 2595) - 1)
    pts = torch.tensor([inv(m) for m in torch.linspace(mel(fmin), mel(fmax), n_mels + 2).tolist()])
    bins = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1)
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for i in range(n_mels):
        lo, c, hi = pts[i], pts[i + 1], pts[i + 2]
        fb[i] = torch.clamp(torch.min((bins - lo) / (c - lo), (hi - bins) / (hi - c)), min=0)
    return fb


def firwin(numtaps: int, cutoff: float, win="hamming") -> torch.Tensor:
    """Low-pass FIR taps; ``cutoff`` as a fraction of the Nyquist frequency."""
    t = torch.arange(numtaps) - (numtaps - 1) / 2
    h = cutoff * torch.sinc(cutoff * t) * window(win, numtaps, periodic=False)
    return h / h.sum()


def lfilter_fir(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    pad = taps.numel() - 1
    y = torch.nn.functional.conv1d(torch.nn.functional.pad(x.reshape(1, 1, -1), (pad, 0)), taps.flip(0).reshape(1, 1, -1).to(x))
    return y.reshape(x.shape)


def resample(x: torch.Tensor, up: int, down: int, taps: int = 63) -> torch.Tensor:
    z = torch.zeros(x.numel() * up, dtype=x.dtype, device=x.device)
    z[::up] = x
    h = firwin(taps, 1.0 / max(up, down)).to(x) * up
    y = torch.nn.functional.conv1d(z.reshape(1, 1, -1), h.reshape(1, 1, -1), padding=taps // 2).reshape(-1)
    return y[::down]


def haar_dwt(x: torch.Tensor):
    x = x[..., : x.shape[-1] // 2 * 2]
    a, b = x[..., 0::2], x[..., 1::2]
    return (a + b) / math.sqrt(2), (a - b) / math.sqrt(2)


def haar_idwt(approx: torch.Tensor, detail: torch.Tensor) -> torch.Tensor:
    out = torch.empty(*approx.shape[:-1], approx.shape[-1] * 2, dtype=approx.dtype, device=approx.device)
    out[..., 0::2], out[..., 1::2] = (approx + detail) / math.sqrt(2), (approx - detail) / math.sqrt(2)
    return out


# ---- spectral family of the functional API (crates/torsh-functional/src/{spectral,spectral_analysis,spectral_stft}.rs) -----
def fft(x, n=None, dim=-1, norm=None): return torch.fft.fft(x, n, dim, norm)
def ifft(x, n=None, dim=-1, norm=None): return torch.fft.ifft(x, n, dim, norm)
def rfft(x, n=None, dim=-1, norm=None): return torch.fft.rfft(x, n, dim, norm)
def irfft(x, n=None, dim=-1, norm=None): return torch.fft.irfft(x, n, dim, norm)
def hfft(x, n=None, dim=-1, norm=None): return torch.fft.hfft(x, n, dim, norm)
def ihfft(x, n=None, dim=-1, norm=None): return torch.fft.ihfft(x, n, dim, norm)
def fft2(x, s=None, dim=(-2, -1), norm=None): return torch.fft.fft2(x, s, dim, norm)
def rfft2(x, s=None, dim=(-2, -1), norm=None): return torch.fft.rfft2(x, s, dim, norm)
def fftn(x, s=None, dim=None, norm=None): return torch.fft.fftn(x, s, dim, norm)
def ifftn(x, s=None, dim=None, norm=None): return torch.fft.ifftn(x, s, dim, norm)
def rfftn(x, s=None, dim=None, norm=None): return torch.fft.rfftn(x, s, dim, norm)
def generate_window(kind: str, n: int, periodic: bool = True, **kw): return window(kind, n, periodic, **kw)


def hz_to_mel(f, htk: bool = True):
    """HTK mel scale (2595 log10(1 + f / 700)); ``htk=False`` gives the Slaney scale (linear below 1 kHz, log above)."""
    f = torch.as_tensor(f, dtype=torch.float64)
    if htk:
        return 2595.0 * torch.log10(1.0 + f / 700.0)
    lin = f / (200.0 / 3)
    log = 15.0 + torch.log(f.clamp_min(1e-10) / 1000.0) / (math.log(6.4) / 27.0)
    return torch.where(f >= 1000.0, log, lin)


def mel_to_hz(m, htk: bool = True):
    m = torch.as_tensor(m, dtype=torch.float64)
    if htk:
        return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    lin = m * (200.0 / 3)
    log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
    return torch.where(m >= 15.0, log, lin)


def create_mel_filterbank(n_mels: int, n_fft: int, sample_rate: int, fmin=0.0, fmax=None) -> torch.Tensor:
    return mel_filterbank(n_mels, n_fft, sample_rate, fmin, fmax)


def mel_spectrogram(x, sample_rate: int, n_fft=512, hop=None, n_mels=80, power=2.0, fmin=0.0, fmax=None, log: bool = False):
    """``[..., n_mels, frames]`` mel-scaled (optionally log) power spectrogram."""
    spec = spectrogram(x, n_fft, hop, power)
    fb = mel_filterbank(n_mels, n_fft, sample_rate, fmin, fmax).to(spec)
    m = fb @ spec
    return torch.log(m.clamp_min(1e-10)) if log else m


def cepstrum(x, n=None, dim=-1):
    """Real cepstrum: inverse FFT of the log magnitude spectrum."""
    X = torch.fft.fft(x, n, dim)
    return torch.fft.ifft(torch.log(X.abs().clamp_min(1e-12)), dim=dim).real


def spectral_centroid(spec: torch.Tensor, sample_rate: int) -> torch.Tensor:
    """Magnitude-weighted mean frequency per frame of a ``[..., bins, frames]`` spectrogram."""
    freqs = torch.linspace(0, sample_rate / 2, spec.shape[-2], device=spec.device, dtype=spec.dtype)
    return (freqs[:, None] * spec).sum(-2) / spec.sum(-2).clamp_min(1e-12)


def spectral_rolloff(spec: torch.Tensor, sample_rate: int, roll_percent: float = 0.85) -> torch.Tensor:
    """Frequency below which ``roll_percent`` of a frame's spectral energy lies."""
    freqs = torch.linspace(0, sample_rate / 2, spec.shape[-2], device=spec.device, dtype=spec.dtype)
    c = spec.cumsum(-2)
    idx = (c >= roll_percent * c[..., -1:, :]).float().argmax(-2)
    return freqs[idx]


def stft_complete(x, n_fft=512, hop=None, win="hann", center=True, normalized: bool = False, onesided: bool = True):
    w = window(win, n_fft).to(x)
    return torch.stft(x, n_fft, hop or n_fft // 4, window=w, center=center, normalized=normalized, onesided=onesided, return_complex=True)


def istft_complete(X, n_fft=512, hop=None, win="hann", center=True, normalized: bool = False, onesided: bool = True, length=None):
    w = window(win, n_fft).to(X.real)
    return torch.istft(X, n_fft, hop or n_fft // 4, window=w, center=center, normalized=normalized, onesided=onesided, length=length)
