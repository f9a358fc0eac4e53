"""Image file IO without external imaging libraries: PNG (8-bit grey / RGB / RGBA, via zlib), binary PPM / PGM, 24-bit
BMP and ``.npy`` tensors; directory / pattern / batch loaders with per-file error reporting, format conversion and image
info. Images are ``uint8`` tensors ``[C, H, W]``. Reference: crates/torsh-vision/src/io.rs (VisionIO and its batch results).
"""
from __future__ import annotations

import fnmatch
import struct
import zlib
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch


# ---- codecs ----------------------------------------------------------------------------------------------------------
def _png_chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def encode_png(img: torch.Tensor) -> bytes:
    c, h, w = img.shape
    color = {1: 0, 3: 2, 4: 6}[c]
    rows = img.permute(1, 2, 0).contiguous().numpy().astype(np.uint8).reshape(h, w * c)
    raw = b"".join(b"\x00" + rows[y].tobytes() for y in range(h))           # filter type 0 on every scan line
    return (b"\x89PNG\r\n\x1a\n" + _png_chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, color, 0, 0, 0))
            + _png_chunk(b"IDAT", zlib.compress(raw, 6)) + _png_chunk(b"IEND", b""))


def decode_png(data: bytes) -> torch.Tensor:
    if data[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("not a PNG file")
    pos, idat, hdr = 8, [], None
    while pos < len(data):
        n, tag = struct.unpack(">I", data[pos:pos + 4])[0], data[pos + 4:pos + 8]
        body = data[pos + 8:pos + 8 + n]
        if tag == b"IHDR":
            hdr = struct.unpack(">IIBBBBB", body)
        elif tag == b"IDAT":
            idat.append(body)
        elif tag == b"IEND":
            break
        pos += 12 + n
    w, h, depth, color, _, _, interlace = hdr
    if depth != 8 or interlace or color not in (0, 2, 6):
        raise ValueError("only 8-bit non-interlaced grey / RGB / RGBA PNG files are supported")
    c = {0: 1, 2: 3, 6: 4}[color]
    raw = zlib.decompress(b"".join(idat))
    stride = w * c
    out = np.zeros((h, stride), dtype=np.uint8)
    prev = np.zeros(stride, dtype=np.int32)
    for y in range(h):
        f = raw[y * (stride + 1)]
        line = np.frombuffer(raw, dtype=np.uint8, count=stride, offset=y * (stride + 1) + 1).astype(np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:
            cur = np.zeros(stride, dtype=np.int32)
            for i in range(stride):
                a = cur[i - c] if i >= c else 0
                b = prev[i]
                cc = prev[i - c] if i >= c else 0
                if f == 1:
                    pred = a
                elif f == 3:
                    pred = (a + b) // 2
                else:                                  # Paeth
                    p = a + b - cc
                    pa, pb, pc = abs(p - a), abs(p - b), abs(p - cc)
                    pred = a if pa <= pb and pa <= pc else (b if pb <= pc else cc)
                cur[i] = (line[i] + pred) & 255
        out[y] = cur
        prev = cur
    return torch.from_numpy(out.reshape(h, w, c)).permute(2, 0, 1).contiguous()


def encode_pnm(img: torch.Tensor) -> bytes:
    c, h, w = img.shape
    if c not in (1, 3):
        raise ValueError("PNM holds 1 or 3 channels")
    return (b"P5" if c == 1 else b"P6") + f"\n{w} {h}\n255\n".encode() + img.permute(1, 2, 0).contiguous().numpy().astype(np.uint8).tobytes()


def decode_pnm(data: bytes) -> torch.Tensor:
    magic = data[:2]
    if magic not in (b"P5", b"P6"):
        raise ValueError("only binary PGM (P5) / PPM (P6) are supported")
    vals, pos = [], 2
    while len(vals) < 3:
        while data[pos:pos + 1].isspace():
            pos += 1
        if data[pos:pos + 1] == b"#":
            pos = data.index(b"\n", pos)
            continue
        end = pos
        while not data[end:end + 1].isspace():
            end += 1
        vals.append(int(data[pos:end]))
        pos = end
    w, h, mx = vals
    if mx != 255:
        raise ValueError("only 8-bit PNM files are supported")
    c = 1 if magic == b"P5" else 3
    arr = np.frombuffer(data, dtype=np.uint8, count=w * h * c, offset=pos + 1)
    return torch.from_numpy(arr.reshape(h, w, c).copy()).permute(2, 0, 1).contiguous()


def encode_bmp(img: torch.Tensor) -> bytes:
    c, h, w = img.shape
    rgb = img.expand(3, h, w) if c == 1 else img[:3]
    rows = rgb.flip(0).permute(1, 2, 0).contiguous().numpy().astype(np.uint8)       # BGR, bottom-up below
    pad = (-w * 3) % 4
    body = b"".join(rows[y].tobytes() + b"\x00" * pad for y in range(h - 1, -1, -1))
    head = struct.pack("<2sIHHI", b"BM", 54 + len(body), 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, w, h, 1, 24, 0, len(body), 2835, 2835, 0, 0)
    return head + body


def decode_bmp(data: bytes) -> torch.Tensor:
    if data[:2] != b"BM":
        raise ValueError("not a BMP file")
    off = struct.unpack("<I", data[10:14])[0]
    w, h, _, bpp, comp = struct.unpack("<iiHHI", data[18:34])
    if bpp != 24 or comp != 0:
        raise ValueError("only uncompressed 24-bit BMP files are supported")
    stride = (w * 3 + 3) // 4 * 4
    flip = h > 0
    h = abs(h)
    arr = np.frombuffer(data, dtype=np.uint8, count=stride * h, offset=off).reshape(h, stride)[:, :w * 3].reshape(h, w, 3)
    if flip:
        arr = arr[::-1]
    return torch.from_numpy(arr[:, :, ::-1].copy()).permute(2, 0, 1).contiguous()


_CODECS = {".png": (encode_png, decode_png), ".ppm": (encode_pnm, decode_pnm), ".pgm": (encode_pnm, decode_pnm), ".bmp": (encode_bmp, decode_bmp)}


# ---- VisionIO --------------------------------------------------------------------------------------------------------
@dataclass
class ImageInfo:
    path: str
    width: int
    height: int
    channels: int
    format: str
    file_size: int


@dataclass
class BatchResult:
    ok: list = field(default_factory=list)            # (path, payload)
    failed: list = field(default_factory=list)        # (path, error message)

    def success_rate(self) -> float:
        n = len(self.ok) + len(self.failed)
        return len(self.ok) / n if n else 1.0

    def all_successful(self) -> bool:
        return not self.failed


class VisionIO:
    def __init__(self, default_format: str = "png", cache_size_mb: int = 0):
        self.default_format = default_format
        self.extensions = set(_CODECS) | {".npy"}
        self._cache, self._cache_bytes, self._cache_cap = {}, 0, cache_size_mb << 20

    def with_caching(self, enable: bool, cache_size_mb: int = 64) -> "VisionIO":
        self._cache_cap = (cache_size_mb << 20) if enable else 0
        return self

    def add_extension(self, ext: str) -> "VisionIO":
        self.extensions.add(ext if ext.startswith(".") else "." + ext)
        return self

    def supported_formats(self) -> list[str]:
        return sorted(e.lstrip(".") for e in _CODECS) + ["npy"]

    def is_supported_image(self, path) -> bool:
        return Path(path).suffix.lower() in self.extensions

    def load_image(self, path) -> torch.Tensor:
        p = Path(path)
        key = (str(p), p.stat().st_mtime_ns)
        if key in self._cache:
            return self._cache[key]
        ext = p.suffix.lower()
        if ext == ".npy":
            img = torch.from_numpy(np.load(p))
        elif ext in _CODECS:
            img = _CODECS[ext][1](p.read_bytes())
        else:
            raise ValueError(f"unsupported image format {ext!r}")
        nbytes = img.numel() * img.element_size()
        if self._cache_cap and self._cache_bytes + nbytes <= self._cache_cap:
            self._cache[key] = img
            self._cache_bytes += nbytes
        return img

    def save_image(self, image: torch.Tensor, path) -> None:
        p = Path(path)
        ext = p.suffix.lower() or "." + self.default_format
        p = p if p.suffix else p.with_suffix(ext)
        img = self.to_uint8(image)
        if ext == ".npy":
            np.save(p, img.numpy())
        elif ext in _CODECS:
            p.write_bytes(_CODECS[ext][0](img))
        else:
            raise ValueError(f"unsupported image format {ext!r}")

    @staticmethod
    def to_uint8(t: torch.Tensor) -> torch.Tensor:
        """Float images in [0, 1] are scaled to 0..255; 2-D tensors gain a channel axis."""
        t = t.detach().cpu()
        if t.dim() == 2:
            t = t[None]
        if t.dtype != torch.uint8:
            t = (t.float().clamp(0, 1) * 255).round().to(torch.uint8)
        return t

    save_tensor_as_image = save_image

    def load_images_from_dir(self, directory, recursive: bool = False) -> BatchResult:
        it = Path(directory).rglob("*") if recursive else Path(directory).iterdir()
        return self.batch_load_images(sorted(p for p in it if p.is_file() and self.is_supported_image(p)))

    def load_images_with_pattern(self, directory, pattern: str) -> BatchResult:
        return self.batch_load_images(sorted(p for p in Path(directory).iterdir() if fnmatch.fnmatch(p.name, pattern)))

    def batch_load_images(self, paths) -> BatchResult:
        r = BatchResult()
        for p in paths:
            try:
                r.ok.append((str(p), self.load_image(p)))
            except Exception as e:
                r.failed.append((str(p), f"{type(e).__name__}: {e}"))
        return r

    def batch_save_images(self, images, directory, prefix: str = "img", fmt: str | None = None) -> BatchResult:
        d = Path(directory)
        d.mkdir(parents=True, exist_ok=True)
        r = BatchResult()
        for i, im in enumerate(images):
            p = d / f"{prefix}_{i:05d}.{fmt or self.default_format}"
            try:
                self.save_image(im, p)
                r.ok.append((str(p), None))
            except Exception as e:
                r.failed.append((str(p), f"{type(e).__name__}: {e}"))
        return r

    def convert_and_save(self, src, dst) -> None:
        self.save_image(self.load_image(src), dst)

    def batch_convert_format(self, paths, out_dir, fmt: str) -> BatchResult:
        d = Path(out_dir)
        d.mkdir(parents=True, exist_ok=True)
        r = BatchResult()
        for p in paths:
            q = d / (Path(p).stem + "." + fmt)
            try:
                self.convert_and_save(p, q)
                r.ok.append((str(q), None))
            except Exception as e:
                r.failed.append((str(p), f"{type(e).__name__}: {e}"))
        return r

    def get_image_info(self, path) -> ImageInfo:
        p = Path(path)
        img = self.load_image(p)
        return ImageInfo(str(p), img.shape[-1], img.shape[-2], img.shape[0], p.suffix.lstrip(".").lower(), p.stat().st_size)


_global_io = VisionIO()


def global_io() -> VisionIO:
    return _global_io


def configure_global_io(io: VisionIO) -> None:
    global _global_io
    _global_io = io
