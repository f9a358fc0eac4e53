"""Signal processing beyond :mod:`torsh_b200.signal` (``crates/torsh-signal/src/{windows,filters,advanced_filters,audio,
resampling,streaming,wavelets}.rs``): the full window family, IIR design (Butterworth, Chebyshev I / II, elliptic through
scipy's pole placement when available, Bessel) by the bilinear transform, ``lfilter`` / ``filtfilt`` / second-order
sections, frequency response and stability analysis, FIR design (``firwin2``, Parks-McClellan style weighted least
squares, Savitzky-Golay), adaptive filters (LMS / NLMS / RLS), cepstra and MFCC, chroma, pitch (autocorrelation, YIN),
perceptual scales, polyphase / sinc / linear resampling, overlap-add and stateful streaming filters, streaming STFT,
lifting wavelets and wavelet packets.  Design code is float64; filters run as tensor ops."""
from __future__ import annotations

import math
import numpy as np
import torch
import torch.nn.functional as F

from . import signal as S
from .nn import functional_ext as X


# ================================================================================================ windows
def _cosine_sum(n, coeffs, periodic):
    m = n if periodic else n - 1
    k = torch.arange(n, dtype=torch.float64)
    return sum((-1) ** i * a * torch.cos(2 * math.pi * i * k / max(m, 1)) for i, a in enumerate(coeffs))


def get_window(kind: str, n: int, periodic: bool = False, **kw) -> torch.Tensor:
    """``hann``, ``hamming``, ``blackman``, ``blackman_harris``, ``nuttall``, ``flat_top``, ``bartlett``, ``bohman``, ``cosine``,
    ``tukey(alpha)``, ``gaussian(std)``, ``exponential(tau)``, ``kaiser(beta)``, ``rectangular`` (float64, symmetric by default)."""
    k = torch.arange(n, dtype=torch.float64)
    m = n if periodic else n - 1
    table = {"hann": [0.5, 0.5], "hamming": [0.54, 0.46], "blackman": [0.42, 0.5, 0.08], "blackman_harris": [0.35875, 0.48829, 0.14128, 0.01168],
             "nuttall": [0.3635819, 0.4891775, 0.1365995, 0.0106411], "flat_top": [0.21557895, 0.41663158, 0.277263158, 0.083578947, 0.006947368]}
    if kind in table:
        return _cosine_sum(n, table[kind], periodic)
    if kind in ("rectangular", "boxcar", "rect"):
        return torch.ones(n, dtype=torch.float64)
    if kind == "bartlett":
        return 1 - (2 * k / max(m, 1) - 1).abs()
    if kind == "cosine":
        return torch.sin(math.pi * (k + 0.5) / n)
    if kind == "bohman":
        x = (2 * k / max(m, 1) - 1).abs()
        w = (1 - x) * torch.cos(math.pi * x) + torch.sin(math.pi * x) / math.pi
        w[0] = w[-1] = 0
        return w
    if kind == "tukey":
        a = kw.get("alpha", 0.5)
        if a <= 0:
            return torch.ones(n, dtype=torch.float64)
        w, edge = torch.ones(n, dtype=torch.float64), a * m / 2
        lo, hi = k < edge, k > m - edge
        w[lo] = 0.5 * (1 + torch.cos(math.pi * (k[lo] / edge - 1)))
        w[hi] = 0.5 * (1 + torch.cos(math.pi * ((k[hi] - m + edge) / edge)))
        return w
    if kind == "gaussian":
        return torch.exp(-0.5 * ((k - m / 2) / kw.get("std", n / 6)) ** 2)
    if kind == "exponential":
        return torch.exp(-(k - m / 2).abs() / kw.get("tau", n / 4))
    if kind == "kaiser":
        return torch.kaiser_window(n, periodic=periodic, beta=kw.get("beta", 12.0), dtype=torch.float64)
    raise ValueError(f"unknown window {kind!r}")


def normalize_window(w, how: str = "amplitude"): return w / (w.sum() if how == "amplitude" else w.pow(2).sum().sqrt())


def kaiser_parameters(ripple_db: float, transition_width: float) -> tuple[int, float]:
    """Kaiser's formulas: filter length and beta for a stop-band attenuation and a transition width (fraction of Nyquist)."""
    a = ripple_db
    beta = 0.1102 * (a - 8.7) if a > 50 else 0.5842 * (a - 21) ** 0.4 + 0.07886 * (a - 21) if a > 21 else 0.0
    return int(math.ceil((a - 7.95) / (2.285 * math.pi * transition_width) + 1)), beta


# ================================================================================================ IIR design
def _analog_prototype(kind, n, rp=None, rs=None):
    if kind == "butter":
        k = np.arange(1, n + 1)
        return np.array([]), np.exp(1j * math.pi * (2 * k + n - 1) / (2 * n)), 1.0
    if kind == "cheby1":
        eps = math.sqrt(10 ** (rp / 10) - 1)
        mu = math.asinh(1 / eps) / n
        th = math.pi * (2 * np.arange(1, n + 1) - 1) / (2 * n)
        p = -np.sinh(mu) * np.sin(th) + 1j * np.cosh(mu) * np.cos(th)
        k = np.real(np.prod(-p))
        return np.array([]), p, k / math.sqrt(1 + eps * eps) if n % 2 == 0 else k
    if kind == "cheby2":
        de = 1 / math.sqrt(10 ** (rs / 10) - 1)
        mu = math.asinh(1 / de) / n
        m = np.arange(-n + 1, n, 2)
        if n % 2:
            m = m[m != 0]
        z = -np.conj(1j / np.sin(m * math.pi / (2 * n)))
        th = math.pi * np.arange(-n + 1, n, 2) / (2 * n)
        p = -np.exp(1j * th)
        p = 1 / (np.sinh(mu) * p.real + 1j * np.cosh(mu) * p.imag)
        return z, p, np.real(np.prod(-p) / np.prod(-z))
    if kind == "bessel":
        # reverse Bessel polynomial roots, normalised to the -3 dB point numerically
        c = [math.factorial(2 * n - k) / (2 ** (n - k) * math.factorial(k) * math.factorial(n - k)) for k in range(n + 1)]
        p = np.roots(c[::-1])
        lo, hi = 0.1, 10.0
        for _ in range(80):
            mid = math.sqrt(lo * hi)
            mag = abs(c[0] / np.polyval(c[::-1], 1j * mid))
            lo, hi = (mid, hi) if mag > 1 / math.sqrt(2) else (lo, mid)
        p = p / mid
        return np.array([]), p, np.real(np.prod(-p))
    raise ValueError(f"unknown filter family {kind!r}")


def _transform(z, p, k, wn, btype):
    """Analog low-pass prototype to low / high / band-pass / band-stop at (pre-warped) ``wn``."""
    deg = len(p) - len(z)
    if btype == "lowpass":
        return z * wn, p * wn, k * wn ** deg
    if btype == "highpass":
        return np.concatenate([wn / z, np.zeros(deg)]), wn / p, k * np.real(np.prod(-z) / np.prod(-p))
    bw, w0 = wn[1] - wn[0], math.sqrt(wn[0] * wn[1])
    if btype == "bandpass":
        zl, pl = z * bw / 2, p * bw / 2
        zz = np.concatenate([zl + np.sqrt(zl ** 2 - w0 ** 2 + 0j), zl - np.sqrt(zl ** 2 - w0 ** 2 + 0j), np.zeros(deg)])
        pp = np.concatenate([pl + np.sqrt(pl ** 2 - w0 ** 2 + 0j), pl - np.sqrt(pl ** 2 - w0 ** 2 + 0j)])
        return zz, pp, k * bw ** deg
    zh, ph = (bw / 2) / z, (bw / 2) / p
    zz = np.concatenate([zh + np.sqrt(zh ** 2 - w0 ** 2 + 0j), zh - np.sqrt(zh ** 2 - w0 ** 2 + 0j), np.full(deg, 1j * w0), np.full(deg, -1j * w0)])
    pp = np.concatenate([ph + np.sqrt(ph ** 2 - w0 ** 2 + 0j), ph - np.sqrt(ph ** 2 - w0 ** 2 + 0j)])
    return zz, pp, k * np.real(np.prod(-z) / np.prod(-p))


def iir_design(order: int, cutoff, btype: str = "lowpass", family: str = "butter", rp: float = 1.0, rs: float = 40.0, output: str = "ba"):
    """Digital IIR filter by the bilinear transform; ``cutoff`` as a fraction of Nyquist (a pair for band filters).
    Returns ``(b, a)`` or second-order sections ``[n, 6]``.  ``elliptic`` uses scipy's analog prototype."""
    if family == "elliptic":
        from scipy import signal as ss
        z, p, k = ss.ellipap(order, rp, rs)
    else:
        z, p, k = _analog_prototype(family, order, rp, rs)
    fs = 2.0
    warped = 2 * fs * np.tan(math.pi * np.asarray(cutoff, dtype=float) / fs)
    z, p, k = _transform(np.asarray(z, complex), np.asarray(p, complex), k, warped if np.ndim(warped) else float(warped), btype)
    fs2 = 2 * fs
    deg = len(p) - len(z)
    zd, pd = (fs2 + z) / (fs2 - z), (fs2 + p) / (fs2 - p)
    kd = k * np.real(np.prod(fs2 - z) / np.prod(fs2 - p))
    zd = np.concatenate([zd, -np.ones(deg)])
    if output == "zpk":
        return zd, pd, kd
    if output == "sos":
        return torch.from_numpy(_zpk2sos(zd, pd, kd))
    return torch.from_numpy(np.real(kd * np.poly(zd))), torch.from_numpy(np.real(np.poly(pd)))


def _pairs(r):
    """Conjugate pairs first (sorted by closeness to the unit circle), then real roots in pairs."""
    r = list(r)
    cplx = sorted([x for x in r if x.imag > 1e-12], key=lambda x: abs(abs(x) - 1))
    real = sorted([x.real for x in r if abs(x.imag) <= 1e-12], key=lambda x: abs(abs(x) - 1))
    out = [(c, np.conj(c)) for c in cplx]
    while len(real) >= 2:
        out.append((real.pop(0), real.pop(0)))
    if real:
        out.append((real.pop(0), None))
    return out


def _zpk2sos(z, p, k):
    pp, zz = _pairs(p), _pairs(z)
    while len(zz) < len(pp):
        zz.append((None, None))
    sos = np.zeros((len(pp), 6))
    for i, ((p1, p2), (z1, z2)) in enumerate(zip(pp, zz)):
        b = np.real(np.poly([r for r in (z1, z2) if r is not None]))
        a = np.real(np.poly([r for r in (p1, p2) if r is not None]))
        sos[i, :len(b)], sos[i, 3:3 + len(a)] = b, a
    sos[0, :3] *= k
    return sos


def butterworth(order, cutoff, btype="lowpass", **kw): return iir_design(order, cutoff, btype, "butter", **kw)
def chebyshev1(order, rp, cutoff, btype="lowpass", **kw): return iir_design(order, cutoff, btype, "cheby1", rp=rp, **kw)
def chebyshev2(order, rs, cutoff, btype="lowpass", **kw): return iir_design(order, cutoff, btype, "cheby2", rs=rs, **kw)
def elliptic(order, rp, rs, cutoff, btype="lowpass", **kw): return iir_design(order, cutoff, btype, "elliptic", rp=rp, rs=rs, **kw)
def bessel(order, cutoff, btype="lowpass", **kw): return iir_design(order, cutoff, btype, "bessel", **kw)


# ================================================================================================ filtering
def lfilter(b, a, x: torch.Tensor, zi: torch.Tensor | None = None, return_state: bool = False):
    """Direct form II transposed along the last axis; ``zi`` is the delay-line state (``max(len(a), len(b)) - 1`` values)."""
    b, a = torch.as_tensor(b, dtype=torch.float64), torch.as_tensor(a, dtype=torch.float64)
    n = max(len(a), len(b))
    b, a = F.pad(b, (0, n - len(b))) / a[0], F.pad(a, (0, n - len(a))) / a[0]
    xd = x.double()
    z = torch.zeros(*xd.shape[:-1], n - 1, dtype=torch.float64) if zi is None else zi.double().clone()
    if n == 1:
        y = b[0] * xd
        return (y.to(x.dtype), z) if return_state else y.to(x.dtype)
    out = []
    for t in range(xd.shape[-1]):
        xt = xd[..., t]
        yt = b[0] * xt + z[..., 0]
        z = torch.cat([z[..., 1:], torch.zeros_like(z[..., :1])], -1) + b[1:] * xt[..., None] - a[1:] * yt[..., None]
        out.append(yt)
    y = torch.stack(out, -1).to(x.dtype)
    return (y, z) if return_state else y


def sosfilt(sos, x):
    for s in torch.as_tensor(sos, dtype=torch.float64):
        x = lfilter(s[:3], s[3:], x)
    return x


def lfilter_zi(b, a) -> torch.Tensor:
    """Delay-line state of the step response's steady state (unit input held for ever)."""
    b, a = np.atleast_1d(np.asarray(b, float)), np.atleast_1d(np.asarray(a, float))
    n = max(len(a), len(b))
    b, a = np.pad(b, (0, n - len(b))) / a[0], np.pad(a, (0, n - len(a))) / a[0]
    comp = np.zeros((n - 1, n - 1))
    comp[0] = -a[1:]
    comp[1:, :-1] = np.eye(n - 2)
    return torch.from_numpy(np.linalg.solve(np.eye(n - 1) - comp.T, b[1:] - a[1:] * b[0]))


def filtfilt(b, a, x: torch.Tensor, padlen: int | None = None):
    """Zero-phase filtering: forward and backward passes over an odd-reflected extension of ``padlen`` samples, each pass
    started from the steady state for its first sample (no start-up transient)."""
    n = max(len(a), len(b))
    padlen = 3 * n if padlen is None else padlen
    left, right = 2 * x[..., :1] - x[..., 1:padlen + 1].flip(-1), 2 * x[..., -1:] - x[..., -padlen - 1:-1].flip(-1)
    ext = torch.cat([left, x, right], -1).double()
    zi = lfilter_zi(b, a)
    y = lfilter(b, a, ext, zi * ext[..., :1])
    y = lfilter(b, a, y.flip(-1), zi * y[..., -1:]).flip(-1)
    return y[..., padlen:ext.shape[-1] - padlen].to(x.dtype)


def freqz(b, a=1.0, n: int = 512):
    """Frequency response at ``n`` points on ``[0, pi)``: ``(w, H)``."""
    w = torch.linspace(0, math.pi, n + 1, dtype=torch.float64)[:-1]
    ejw = torch.exp(-1j * w)
    poly = lambda c: sum(ck * ejw ** k for k, ck in enumerate(torch.atleast_1d(torch.as_tensor(c, dtype=torch.float64)).to(torch.complex128)))
    return w, poly(b) / poly(a)


def group_delay(b, a=1.0, n: int = 512):
    w, h = freqz(b, a, n)
    ph = torch.from_numpy(np.unwrap(torch.angle(h).numpy()))
    return w[:-1], -(ph[1:] - ph[:-1]) / (w[1] - w[0])


def impulse_response(b, a=1.0, n: int = 64): imp = torch.zeros(n, dtype=torch.float64); imp[0] = 1; return lfilter(b, a, imp)
def is_stable(a) -> bool: c = np.atleast_1d(np.asarray(a, dtype=float)); return bool(np.all(np.abs(np.roots(c)) < 1)) if len(c) > 1 else True


def stability_analysis(b, a) -> dict:
    poles, zeros = np.roots(np.atleast_1d(np.asarray(a, float))), np.roots(np.atleast_1d(np.asarray(b, float)))
    return {"stable": bool(np.all(np.abs(poles) < 1)), "max_pole_radius": float(np.abs(poles).max()) if len(poles) else 0.0,
            "minimum_phase": bool(np.all(np.abs(zeros) <= 1 + 1e-9)), "poles": poles, "zeros": zeros}


def firwin2(numtaps: int, freqs, gains, window: str = "hamming") -> torch.Tensor:
    """Linear-phase FIR from a piecewise-linear magnitude by frequency sampling and windowing (odd ``numtaps``)."""
    nfreqs = 1 + 2 ** int(math.ceil(math.log2(numtaps)))
    grid = np.linspace(0, 1, nfreqs)
    mag = np.interp(grid, freqs, gains)
    shift = np.exp(-1j * math.pi * grid * (numtaps - 1) / 2)
    h = np.fft.irfft(mag * shift)[:numtaps]
    return torch.from_numpy(h) * get_window(window, numtaps)


def remez(numtaps: int, bands, desired, weights=None, grid: int = 16) -> torch.Tensor:
    """Weighted least-squares design of a type I linear-phase FIR on a dense grid of the bands (fractions of Nyquist) —
    the least-squares counterpart of the Parks-McClellan exchange (same specification format)."""
    m = (numtaps - 1) // 2
    ws, ds, wt = [], [], []
    for i in range(len(bands) // 2):
        pts = np.linspace(bands[2 * i], bands[2 * i + 1], max(grid * m // (len(bands) // 2), 8))
        ws.append(pts); ds.append(np.full_like(pts, desired[i])); wt.append(np.full_like(pts, (weights[i] if weights is not None else 1.0)))
    w, d, g = np.concatenate(ws) * math.pi, np.concatenate(ds), np.sqrt(np.concatenate(wt))
    A = np.cos(np.outer(w, np.arange(m + 1)))
    c = np.linalg.lstsq(A * g[:, None], d * g, rcond=None)[0]
    h = np.concatenate([c[:0:-1] / 2, [c[0]], c[1:] / 2])
    return torch.from_numpy(h)


def savgol_coeffs(window: int, polyorder: int, deriv: int = 0) -> torch.Tensor:
    half = window // 2
    A = np.vander(np.arange(-half, half + 1), polyorder + 1, increasing=True)
    return torch.from_numpy(np.linalg.pinv(A)[deriv] * math.factorial(deriv))


def savgol_filter(x: torch.Tensor, window: int, polyorder: int, deriv: int = 0) -> torch.Tensor:
    """Polynomial smoothing (or differentiation); the ends are fitted with the same polynomial order over the edge window."""
    c = savgol_coeffs(window, polyorder, deriv).to(x)
    half = window // 2
    y = F.conv1d(x.reshape(-1, 1, x.shape[-1]), c.reshape(1, 1, -1), padding=half).reshape(x.shape).clone()
    t = torch.arange(window, dtype=x.dtype)
    V = torch.stack([t ** k for k in range(polyorder + 1)], 1)
    for sl, pos in ((slice(0, window), t[:half]), (slice(-window, None), t[-half:])):
        coef = torch.linalg.lstsq(V, x[..., sl].reshape(-1, window).t()).solution          # [order+1, batch]
        dv = torch.stack([math.factorial(k) / math.factorial(k - deriv) * pos ** (k - deriv) if k >= deriv else torch.zeros_like(pos) for k in range(polyorder + 1)], 1)
        edge = (dv @ coef).t().reshape(*x.shape[:-1], half)
        if sl.start == 0:
            y[..., :half] = edge
        else:
            y[..., -half:] = edge
    return y


def median_filter1d(x, size: int = 3): return F.pad(x.reshape(-1, 1, x.shape[-1]), (size // 2, size // 2), mode="replicate").unfold(-1, size, 1).median(-1).values.reshape(x.shape)
def convolve1d(x, k, mode="full"): return torch.from_numpy(np.convolve(np.asarray(x, float), np.asarray(k, float), mode))
def correlate1d(x, k, mode="full"): return torch.from_numpy(np.correlate(np.asarray(x, float), np.asarray(k, float), mode))


# ================================================================================================ adaptive filters
def lms_filter(x, d, taps: int = 16, mu: float = 0.01, normalized: bool = False, eps: float = 1e-8):
    """Adapts ``w`` so that ``w . [x_t, x_{t-1}, ...]`` tracks ``d``; returns ``(output, error, final weights)``."""
    x, d = np.asarray(x, float), np.asarray(d, float)
    w, y, e = np.zeros(taps), np.zeros(len(x)), np.zeros(len(x))
    buf = np.zeros(taps)
    for t in range(len(x)):
        buf = np.roll(buf, 1); buf[0] = x[t]
        y[t] = w @ buf
        e[t] = d[t] - y[t]
        w += (mu / (eps + buf @ buf) if normalized else mu) * e[t] * buf
    return torch.from_numpy(y), torch.from_numpy(e), torch.from_numpy(w)


def nlms_filter(x, d, taps=16, mu=0.5): return lms_filter(x, d, taps, mu, normalized=True)


def rls_filter(x, d, taps: int = 16, lam: float = 0.99, delta: float = 100.0):
    x, d = np.asarray(x, float), np.asarray(d, float)
    w, P, buf = np.zeros(taps), np.eye(taps) * delta, np.zeros(taps)
    y, e = np.zeros(len(x)), np.zeros(len(x))
    for t in range(len(x)):
        buf = np.roll(buf, 1); buf[0] = x[t]
        k = P @ buf / (lam + buf @ P @ buf)
        y[t] = w @ buf
        e[t] = d[t] - y[t]
        w += k * e[t]
        P = (P - np.outer(k, buf @ P)) / lam
    return torch.from_numpy(y), torch.from_numpy(e), torch.from_numpy(w)


# ================================================================================================ audio features
def hz_to_bark(f): f = torch.as_tensor(f, dtype=torch.float64); return 6 * torch.asinh(f / 600)
def bark_to_hz(b): b = torch.as_tensor(b, dtype=torch.float64); return 600 * torch.sinh(b / 6)
def hz_to_erb(f): f = torch.as_tensor(f, dtype=torch.float64); return 21.4 * torch.log10(1 + 0.00437 * f)
def erb_to_hz(e): e = torch.as_tensor(e, dtype=torch.float64); return (10 ** (e / 21.4) - 1) / 0.00437
def zero_crossing_rate(x): return ((x[..., :-1] * x[..., 1:]) < 0).double().mean(-1)
def real_cepstrum(x): return torch.fft.ifft(torch.log(torch.fft.fft(x.double()).abs().clamp(min=1e-12))).real
def power_cepstrum(x): return torch.fft.ifft(torch.log(torch.fft.fft(x.double()).abs().pow(2).clamp(min=1e-24))).abs() ** 2


def complex_cepstrum(x):
    sp = torch.fft.fft(x.double())
    ph = torch.from_numpy(np.unwrap(torch.angle(sp).numpy()))
    n = len(x)
    ndelay = round(float(ph[(n + 1) // 2]) / math.pi)
    ph = ph - math.pi * ndelay * torch.arange(n, dtype=torch.float64) / ((n + 1) // 2)
    return torch.fft.ifft(torch.log(sp.abs().clamp(min=1e-12)) + 1j * ph).real, ndelay


def minimum_phase(h: torch.Tensor, n_fft: int | None = None) -> torch.Tensor:
    """Minimum-phase FIR with the magnitude of ``h`` (homomorphic method: fold the real cepstrum)."""
    n_fft = n_fft or 2 ** int(math.ceil(math.log2(8 * len(h))))
    c = torch.fft.ifft(torch.log(torch.fft.fft(h.double(), n_fft).abs().clamp(min=1e-10))).real
    fold = torch.zeros(n_fft, dtype=torch.float64)
    fold[0], fold[1:n_fft // 2], fold[n_fft // 2] = c[0], 2 * c[1:n_fft // 2], c[n_fft // 2]
    return torch.fft.ifft(torch.exp(torch.fft.fft(fold))).real[:len(h)]


def dct2(x: torch.Tensor, norm: str = "ortho") -> torch.Tensor:
    n = x.shape[-1]
    k = torch.arange(n, dtype=x.dtype)
    basis = torch.cos(math.pi / n * (k[None] + 0.5) * k[:, None])
    y = x @ basis.t() * 2
    if norm == "ortho":
        y = y * math.sqrt(1 / (2 * n))
        y[..., 0] = y[..., 0] / math.sqrt(2)
    return y


def compute_mfcc(x: torch.Tensor, sample_rate: int, n_mfcc: int = 13, n_mels: int = 40, n_fft: int = 512, hop: int = 160, lifter: int = 0) -> torch.Tensor:
    """``[frames, n_mfcc]``: power spectrogram -> mel filter bank -> log -> DCT-II (optionally liftered)."""
    spec = S.stft(x.float(), n_fft, hop).abs() ** 2                                     # [freq, frames]
    fb = S.mel_filterbank(n_mels, n_fft, sample_rate)
    logmel = torch.log((fb.to(spec) @ spec).clamp(min=1e-10)).t()
    c = dct2(logmel)[:, :n_mfcc]
    if lifter > 0:
        c = c * (1 + lifter / 2 * torch.sin(math.pi * torch.arange(n_mfcc) / lifter))
    return c


def chroma_features(x: torch.Tensor, sample_rate: int, n_fft: int = 2048, hop: int = 512, tuning: float = 440.0) -> torch.Tensor:
    """``[12, frames]`` energy per pitch class (C = row 0), columns normalised to unit maximum."""
    spec = S.stft(x.float(), n_fft, hop).abs() ** 2
    freqs = torch.arange(spec.shape[0]) * sample_rate / n_fft
    pc = (torch.round(12 * torch.log2(freqs[1:] / tuning)).long() + 9) % 12
    m = torch.zeros(12, spec.shape[0]).index_put_((pc, torch.arange(1, spec.shape[0])), torch.ones(len(pc)))
    m[:, freqs < 50] = 0
    c = m @ spec
    return c / c.amax(0, keepdim=True).clamp(min=1e-12)


def autocorr_pitch(x: torch.Tensor, sample_rate: int, fmin: float = 50.0, fmax: float = 1000.0) -> float:
    xd = x.double() - x.double().mean()
    n = len(xd)
    ac = torch.fft.irfft(torch.fft.rfft(xd, 2 * n).abs() ** 2)[:n]
    lo, hi = int(sample_rate / fmax), min(int(sample_rate / fmin), n - 1)
    lag = lo + int(ac[lo:hi].argmax())
    return sample_rate / _parabolic(ac, lag)


def _parabolic(v, i):
    if i <= 0 or i >= len(v) - 1:
        return float(i)
    a, b, c = float(v[i - 1]), float(v[i]), float(v[i + 1])
    den = a - 2 * b + c
    return i + (0.5 * (a - c) / den if den else 0.0)


def yin_pitch(x: torch.Tensor, sample_rate: int, fmin: float = 50.0, fmax: float = 1000.0, threshold: float = 0.1) -> tuple[float, float]:
    """YIN: cumulative-mean-normalised difference function, first dip under ``threshold``, parabolic refinement.
    Returns ``(frequency, aperiodicity)``; frequency 0 when no dip qualifies."""
    xd = x.double()
    n = len(xd)
    tmax = min(int(sample_rate / fmin), n // 2)
    w = n - tmax
    sq = torch.cat([torch.zeros(1, dtype=torch.float64), (xd * xd).cumsum(0)])
    ac = torch.fft.irfft(torch.fft.rfft(xd[:w], 2 * n).conj() * torch.fft.rfft(xd, 2 * n))[:tmax + 1]
    taus = torch.arange(tmax + 1)
    d = sq[w] - sq[0] + (sq[taus + w] - sq[taus]) - 2 * ac
    cm = torch.ones(tmax + 1, dtype=torch.float64)
    cm[1:] = d[1:] * torch.arange(1, tmax + 1) / d[1:].cumsum(0).clamp(min=1e-12)
    lo = max(int(sample_rate / fmax), 2)
    below = (cm[lo:] < threshold).nonzero()
    if len(below) == 0:
        return 0.0, float(cm[lo:].min())
    t = lo + int(below[0])
    while t + 1 <= tmax and cm[t + 1] < cm[t]:
        t += 1
    return sample_rate / _parabolic(cm, t), float(cm[t])


# ================================================================================================ resampling
def linear_resample(x: torch.Tensor, ratio: float) -> torch.Tensor:
    n = int(round(x.shape[-1] * ratio))
    return F.interpolate(x.reshape(-1, 1, x.shape[-1]).double(), size=n, mode="linear", align_corners=True).reshape(*x.shape[:-1], n).to(x.dtype)


def polyphase_resample(x: torch.Tensor, up: int, down: int, taps_per_phase: int = 10, beta: float = 5.0) -> torch.Tensor:
    """Rational rate change ``up / down``: zero-stuffing, Kaiser-windowed sinc low-pass at ``min(1/up, 1/down)``, decimation —
    evaluated as one strided convolution so the stuffed zeros are never multiplied."""
    g = math.gcd(up, down)
    up, down = up // g, down // g
    if up == down == 1:
        return x.clone()
    half = taps_per_phase * max(up, down)
    t = torch.arange(-half, half + 1, dtype=torch.float64)
    fc = 1.0 / max(up, down)
    h = fc * torch.sinc(fc * t) * torch.kaiser_window(2 * half + 1, periodic=False, beta=beta, dtype=torch.float64) * up
    xd = x.reshape(-1, 1, x.shape[-1]).double()
    stuffed = torch.zeros(xd.shape[0], 1, xd.shape[-1] * up, dtype=torch.float64)
    stuffed[..., ::up] = xd
    y = F.conv1d(F.pad(stuffed, (half, half)), h.flip(0).reshape(1, 1, -1), stride=down)
    n_out = int(math.ceil(x.shape[-1] * up / down))
    return y[..., :n_out].reshape(*x.shape[:-1], -1).to(x.dtype)


def sinc_resample(x: torch.Tensor, ratio: float, half_width: int = 16) -> torch.Tensor:
    """Arbitrary-ratio band-limited interpolation: every output sample is a Hann-windowed sinc sum over ``2 * half_width`` inputs."""
    n_out = int(round(x.shape[-1] * ratio))
    pos = torch.arange(n_out, dtype=torch.float64) / ratio
    base = torch.floor(pos).long()
    k = torch.arange(-half_width + 1, half_width + 1)
    idx = (base[:, None] + k[None]).clamp(0, x.shape[-1] - 1)
    t = pos[:, None] - (base[:, None] + k[None]).double()
    fc = min(1.0, ratio)
    w = fc * torch.sinc(fc * t) * (0.5 + 0.5 * torch.cos(math.pi * t / half_width)).clamp(min=0)
    return (x.double()[..., idx] * w).sum(-1).to(x.dtype)


def decimate(x: torch.Tensor, q: int, order: int = 8) -> torch.Tensor:
    b, a = chebyshev1(order, 0.05, 0.8 / q)
    return filtfilt(b, a, x.double())[..., ::q].to(x.dtype)


# ================================================================================================ streaming
class RingBuffer:
    def __init__(self, capacity: int): self.buf, self.capacity, self.head, self.size = torch.zeros(capacity, dtype=torch.float64), capacity, 0, 0
    def __len__(self): return self.size
    def is_full(self): return self.size == self.capacity

    def push(self, x):
        for v in torch.atleast_1d(torch.as_tensor(x, dtype=torch.float64)):
            self.buf[(self.head + self.size) % self.capacity] = v
            if self.size < self.capacity:
                self.size += 1
            else:
                self.head = (self.head + 1) % self.capacity

    def pop(self, n: int) -> torch.Tensor:
        n = min(n, self.size)
        out = self.buf[(self.head + torch.arange(n)) % self.capacity].clone()
        self.head, self.size = (self.head + n) % self.capacity, self.size - n
        return out

    def peek(self): return self.buf[(self.head + torch.arange(self.size)) % self.capacity].clone()


class StreamingFilter:
    """Chunk-by-chunk IIR / FIR filtering that carries the delay-line state, so the concatenated outputs equal one call
    of :func:`lfilter` on the whole signal."""

    def __init__(self, b, a=1.0): self.b, self.a, self.state = torch.atleast_1d(torch.as_tensor(b, dtype=torch.float64)), torch.atleast_1d(torch.as_tensor(a, dtype=torch.float64)), None
    def reset(self): self.state = None

    def process(self, chunk: torch.Tensor) -> torch.Tensor:
        y, self.state = lfilter(self.b, self.a, chunk, self.state, return_state=True)
        return y


class OverlapAddProcessor:
    """FIR filtering of a stream by FFT blocks: each block's linear convolution tail is added to the next block's head."""

    def __init__(self, h: torch.Tensor, block: int = 256):
        self.h, self.block, self.m = h.double(), block, len(h)
        self.nfft = 2 ** int(math.ceil(math.log2(block + self.m - 1)))
        self.H, self.tail = torch.fft.rfft(self.h, self.nfft), torch.zeros(self.m - 1, dtype=torch.float64)

    def process(self, chunk: torch.Tensor) -> torch.Tensor:
        out = []
        for s in range(0, len(chunk), self.block):
            blk = chunk[s:s + self.block].double()
            y = torch.fft.irfft(torch.fft.rfft(blk, self.nfft) * self.H, self.nfft)[:len(blk) + self.m - 1]
            y[:self.m - 1] += self.tail
            out.append(y[:len(blk)])
            tail = y[len(blk):]
            self.tail = F.pad(tail, (0, self.m - 1 - len(tail)))
        return torch.cat(out) if out else torch.zeros(0, dtype=torch.float64)

    def flush(self) -> torch.Tensor: t, self.tail = self.tail, torch.zeros(self.m - 1, dtype=torch.float64); return t


class StreamingSTFT:
    """Frames arrive as soon as ``n_fft`` samples are buffered; hop-size advance; matches ``torch.stft(center=False)``."""

    def __init__(self, n_fft: int = 512, hop: int | None = None, window: str = "hann"):
        self.n_fft, self.hop = n_fft, hop or n_fft // 4
        self.win, self.buf = get_window(window, n_fft, periodic=True), torch.zeros(0, dtype=torch.float64)

    def push(self, chunk: torch.Tensor) -> torch.Tensor:
        self.buf = torch.cat([self.buf, chunk.double()])
        frames = []
        while len(self.buf) >= self.n_fft:
            frames.append(torch.fft.rfft(self.buf[:self.n_fft] * self.win))
            self.buf = self.buf[self.hop:]
        return torch.stack(frames, 1) if frames else torch.zeros(self.n_fft // 2 + 1, 0, dtype=torch.complex128)


def process_chunked(fn, x: torch.Tensor, chunk: int, overlap: int = 0) -> torch.Tensor:
    """Applies a length-preserving ``fn`` to overlapping chunks and keeps each chunk's centre (bounded memory)."""
    out, n, s = [], x.shape[-1], 0
    while s < n:
        lo, hi = max(0, s - overlap), min(n, s + chunk + overlap)
        y = fn(x[..., lo:hi])
        out.append(y[..., s - lo:s - lo + min(chunk, n - s)])
        s += chunk
    return torch.cat(out, -1)


# ================================================================================================ wavelets: lifting and packets
def _fit(v: torch.Tensor, n: int, mode: str = "replicate") -> torch.Tensor:
    """Extends the last axis to ``n`` entries (odd-length signals have one more even than odd sample)."""
    if v.shape[-1] >= n:
        return v[..., :n]
    return torch.cat([v, (v[..., -1:] if mode == "replicate" else torch.zeros_like(v[..., -1:])).expand(*v.shape[:-1], n - v.shape[-1])], -1)


def lifting_dwt(x: torch.Tensor, wavelet: str = "cdf53"):
    """One level by lifting steps: ``haar`` or the LeGall 5/3 biorthogonal wavelet with symmetric extension; any length.
    Returns ``(approximation, detail)``."""
    e, o = x[..., ::2].clone(), x[..., 1::2].clone()
    ne, no = e.shape[-1], o.shape[-1]
    if wavelet == "haar":
        d = o - e[..., :no]
        return e + _fit(d, ne, "zero") / 2, d
    e_next = torch.cat([e[..., 1:], e[..., -1:]], -1)
    d = o - (e[..., :no] + e_next[..., :no]) / 2
    d_prev = torch.cat([d[..., :1], d[..., :-1]], -1)
    return e + (_fit(d_prev, ne) + _fit(d, ne)) / 4, d


def lifting_idwt(a: torch.Tensor, d: torch.Tensor, wavelet: str = "cdf53") -> torch.Tensor:
    ne, no = a.shape[-1], d.shape[-1]
    if wavelet == "haar":
        e = a - _fit(d, ne, "zero") / 2
        o = d + e[..., :no]
    else:
        d_prev = torch.cat([d[..., :1], d[..., :-1]], -1)
        e = a - (_fit(d_prev, ne) + _fit(d, ne)) / 4
        e_next = torch.cat([e[..., 1:], e[..., -1:]], -1)
        o = d + (e[..., :no] + e_next[..., :no]) / 2
    out = torch.zeros(*a.shape[:-1], ne + no, dtype=a.dtype)
    out[..., ::2], out[..., 1::2] = e, o
    return out


def wavelet_packet(x: torch.Tensor, wavelet: str = "db2", level: int = 3) -> dict[str, torch.Tensor]:
    """Full wavelet packet tree: keys are paths of ``a`` / ``d`` (``""`` is the signal); both branches split at every level."""
    tree = {"": x}
    for l in range(level):
        for path in [p for p in tree if len(p) == l]:
            a, d = X.dwt_1d(tree[path], wavelet)
            tree[path + "a"], tree[path + "d"] = a, d
    return tree


def wavelet_packet_reconstruct(tree: dict, wavelet: str = "db2", level: int | None = None) -> torch.Tensor:
    level = max(len(p) for p in tree) if level is None else level
    cur = {p: v for p, v in tree.items() if len(p) == level}
    for l in range(level, 0, -1):
        cur = {p[:-1]: X.idwt_1d(cur[p[:-1] + "a"], cur[p[:-1] + "d"], wavelet) for p in cur if p.endswith("a")}
    return cur[""]


def best_basis(tree: dict, cost=lambda v: float(-(v.pow(2) / v.pow(2).sum().clamp(min=1e-300) * torch.log((v.pow(2) / v.pow(2).sum().clamp(min=1e-300)).clamp(min=1e-300))).sum())) -> list[str]:
    """Coifman-Wickerhauser search: keep a node when its cost (Shannon entropy of normalised energies by default) is no
    more than the best cost of its children."""
    level = max(len(p) for p in tree)
    best = {p: (cost(tree[p]) * float(tree[p].pow(2).sum()), [p]) for p in tree if len(p) == level}
    for l in range(level - 1, -1, -1):
        for p in [q for q in tree if len(q) == l]:
            own = cost(tree[p]) * float(tree[p].pow(2).sum())
            kids = best[p + "a"][0] + best[p + "d"][0]
            best[p] = (own, [p]) if own <= kids else (kids, best[p + "a"][1] + best[p + "d"][1])
    return best[""][1]


def scalogram(x, scales, wavelet="morlet"): return X.cwt(x, scales, wavelet).abs() ** 2
def scale_to_frequency(scale, w0: float = 6.0, dt: float = 1.0): return w0 / (2 * math.pi * scale * dt)
def frequency_to_scale(freq, w0: float = 6.0, dt: float = 1.0): return w0 / (2 * math.pi * freq * dt)
def cone_of_influence(n: int, scale: float) -> tuple[int, int]: e = int(math.ceil(math.sqrt(2) * scale)); return e, n - e
