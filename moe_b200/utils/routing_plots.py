"""Routing snapshot plots as PNG files, with no plotting library.

Same three pictures and file names as the reference (`src/utils/routing_plots.py:21-132`):
`step_XXXXXXXX_layer_heatmap.png` (layers x experts token fraction), and for the global layout
`..._global_fracs.png` (per-expert token fraction bars, red above twice the ideal, ideal line) and
`..._usage_vs_tokens.png` (layers-using-expert vs token fraction scatter with a least-squares
trend line).  Rasterised on the CPU into an RGB array and written with a small PNG encoder
(zlib + CRC from the standard library); axis labels are drawn with a 5x7 bitmap font.
"""
from __future__ import annotations

import os
import struct
import zlib

import numpy as np

_FONT = {
    "0": "01110 10001 10011 10101 11001 10001 01110", "1": "00100 01100 00100 00100 00100 00100 01110",
    "2": "01110 10001 00001 00010 00100 01000 11111", "3": "11110 00001 00001 01110 00001 00001 11110",
    "4": "00010 00110 01010 10010 11111 00010 00010", "5": "11111 10000 11110 00001 00001 10001 01110",
    "6": "00110 01000 10000 11110 10001 10001 01110", "7": "11111 00001 00010 00100 01000 01000 01000",
    "8": "01110 10001 10001 01110 10001 10001 01110", "9": "01110 10001 10001 01111 00001 00010 01100",
    ".": "00000 00000 00000 00000 00000 01100 01100", "-": "00000 00000 00000 11111 00000 00000 00000",
    "=": "00000 00000 11111 00000 11111 00000 00000", " ": "00000 00000 00000 00000 00000 00000 00000",
    "e": "00000 00000 01110 10001 11111 10000 01110", "E": "11111 10000 10000 11110 10000 10000 11111",
    "L": "10000 10000 10000 10000 10000 10000 11111", "s": "00000 00000 01111 10000 01110 00001 11110",
    "t": "01000 01000 11100 01000 01000 01001 00110", "p": "00000 00000 11110 10001 11110 10000 10000",
    "x": "00000 00000 10001 01010 00100 01010 10001", "a": "00000 00000 01110 00001 01111 10001 01111",
    "y": "00000 00000 10001 10001 01111 00001 01110", "r": "00000 00000 10110 11001 10000 10000 10000",
    "f": "00110 01001 01000 11100 01000 01000 01000", "c": "00000 00000 01110 10000 10000 10001 01110",
    "i": "00100 00000 01100 00100 00100 00100 01110", "d": "00001 00001 01101 10011 10001 10001 01111",
    "l": "01100 00100 00100 00100 00100 00100 01110", "o": "00000 00000 01110 10001 10001 10001 01110",
    "n": "00000 00000 10110 11001 10001 10001 10001", "u": "00000 00000 10001 10001 10001 10011 01101",
    "g": "00000 01111 10001 10001 01111 00001 01110", "k": "10000 10000 10010 10100 11000 10100 10010",
    "(": "00010 00100 01000 01000 01000 00100 00010", ")": "01000 00100 00010 00010 00010 00100 01000",
    ",": "00000 00000 00000 00000 01100 00100 01000", "T": "11111 00100 00100 00100 00100 00100 00100",
    "F": "11111 10000 10000 11110 10000 10000 10000", "P": "11110 10001 10001 11110 10000 10000 10000",
    "G": "01110 10001 10000 10111 10001 10001 01111", "U": "10001 10001 10001 10001 10001 10001 01110",
    "I": "01110 00100 00100 00100 00100 00100 01110", "S": "01111 10000 10000 01110 00001 00001 11110",
}


def write_png(path: str, rgb: np.ndarray) -> None:
    """`rgb`: uint8 array `[H, W, 3]`."""
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    png = (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
           + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))
    with open(path, "wb") as f:
        f.write(png)


class Canvas:
    def __init__(self, w: int, h: int):
        self.img = np.full((h, w, 3), 255, dtype=np.uint8)
        self.w, self.h = w, h

    def rect(self, x0, y0, x1, y1, color):
        x0, x1 = sorted((int(x0), int(x1)))
        y0, y1 = sorted((int(y0), int(y1)))
        self.img[max(0, y0):min(self.h, y1 + 1), max(0, x0):min(self.w, x1 + 1)] = color

    def line(self, x0, y0, x1, y1, color, dash: int = 0):
        n = int(max(abs(x1 - x0), abs(y1 - y0))) + 1
        for i, t in enumerate(np.linspace(0, 1, n)):
            if dash and (i // dash) % 2:
                continue
            x, y = int(round(x0 + (x1 - x0) * t)), int(round(y0 + (y1 - y0) * t))
            if 0 <= x < self.w and 0 <= y < self.h:
                self.img[y, x] = color

    def dot(self, x, y, r, color):
        self.rect(x - r, y - r, x + r, y + r, color)

    def text(self, x, y, s: str, color=(0, 0, 0), scale: int = 1):
        for ch in s:
            glyph = _FONT.get(ch) or _FONT.get(ch.lower()) or _FONT.get(ch.upper()) or _FONT[" "]
            for r, row in enumerate(glyph.split()):
                for c, bit in enumerate(row):
                    if bit == "1":
                        self.rect(x + c * scale, y + r * scale, x + (c + 1) * scale - 1, y + (r + 1) * scale - 1, color)
            x += 6 * scale

    def axes(self, x0, y0, x1, y1):
        self.line(x0, y1, x1, y1, (0, 0, 0))
        self.line(x0, y0, x0, y1, (0, 0, 0))


def _heat(v: np.ndarray) -> np.ndarray:
    """Yellow -> orange -> red colour ramp for values in [0, 1]."""
    v = np.clip(v, 0, 1)[..., None]
    lo, mid, hi = np.array([255, 255, 204.0]), np.array([253, 141, 60.0]), np.array([128, 0, 38.0])
    out = np.where(v < 0.5, lo + (mid - lo) * (v * 2), mid + (hi - mid) * (v * 2 - 1))
    return out.astype(np.uint8)


def plot_routing_snapshot(snapshot: dict, output_dir: str, step: int) -> list[str]:
    """Writes the PNGs next to the JSON snapshot; returns the paths written."""
    prefix = os.path.join(output_dir, f"step_{step:08d}")
    written = []
    p = _plot_layer_heatmap(snapshot["layers"], prefix, step)
    if p:
        written.append(p)
    gp = snapshot.get("global_pool")
    if gp is not None:
        written.append(_plot_global_fracs(gp, prefix, step))
        written.append(_plot_usage_vs_tokens(gp, prefix, step))
    return written


def _plot_layer_heatmap(layers: dict, prefix: str, step: int) -> str | None:
    keys = sorted(layers.keys(), key=int)
    if not keys:
        return None
    data = np.array([layers[k]["token_fracs"] for k in keys], dtype=np.float64)
    L, E = data.shape
    cw = max(2, min(12, 1200 // max(E, 1)))
    chh = max(8, min(24, 600 // max(L, 1)))
    ml, mt, mr, mb = 50, 30, 20, 30
    cv = Canvas(ml + E * cw + mr, mt + L * chh + mb)
    vmax = data.max() if data.max() > 0 else 1.0
    colors = _heat(data / vmax)
    for i in range(L):
        for j in range(E):
            cv.rect(ml + j * cw, mt + i * chh, ml + (j + 1) * cw - 1, mt + (i + 1) * chh - 1, colors[i, j])
        cv.text(8, mt + i * chh + max(0, (chh - 7) // 2), str(keys[i]))
    cv.text(ml, 8, f"layer x expert token fraction  step {step}  ideal={1.0 / E:.4f}")
    for j in range(0, E, max(1, E // 10)):
        cv.text(ml + j * cw, mt + L * chh + 8, str(j))
    path = f"{prefix}_layer_heatmap.png"
    write_png(path, cv.img)
    return path


def _plot_global_fracs(gp: dict, prefix: str, step: int) -> str:
    fr = np.array(gp["token_fracs"], dtype=np.float64)
    E = len(fr)
    ideal = 1.0 / max(E, 1)
    bw = max(1, min(8, 1400 // max(E, 1)))
    ml, mt, mr, mb, ph = 60, 30, 20, 30, 300
    cv = Canvas(ml + E * bw + mr, mt + ph + mb)
    top = max(fr.max() if E else 0, ideal * 1.2, 1e-12)
    for j, f in enumerate(fr):
        color = (231, 76, 60) if f > 2 * ideal else (52, 152, 219)
        cv.rect(ml + j * bw, mt + ph - int(ph * f / top), ml + (j + 1) * bw - 1, mt + ph, color)
    cv.axes(ml, mt, ml + E * bw, mt + ph)
    yi = mt + ph - int(ph * ideal / top)
    cv.line(ml, yi, ml + E * bw, yi, (0, 0, 0), dash=4)
    cv.text(ml, 8, f"global pool token fraction  step {step}  ideal={ideal:.4f}")
    cv.text(4, mt, f"{top:.4f}")
    for j in range(0, E, max(1, E // 10)):
        cv.text(ml + j * bw, mt + ph + 8, str(j))
    path = f"{prefix}_global_fracs.png"
    write_png(path, cv.img)
    return path


def _plot_usage_vs_tokens(gp: dict, prefix: str, step: int) -> str:
    fr = np.array(gp["token_fracs"], dtype=np.float64)
    use = np.array(gp["layer_usage_count"], dtype=np.float64)
    nl = gp["num_layers"]
    ml, mt, mr, mb, pw, ph = 70, 30, 20, 40, 520, 360
    cv = Canvas(ml + pw + mr, mt + ph + mb)
    top = max(fr.max() if len(fr) else 0, 1e-12) * 1.1
    sx = lambda u: ml + int(pw * u / max(nl, 1))
    sy = lambda f: mt + ph - int(ph * f / top)
    for u, f in zip(use, fr):
        cv.dot(sx(u), sy(f), 2, (44, 62, 80))
    if len(use) > 2 and use.std() > 0:
        a, b = np.polyfit(use, fr, 1)
        cv.line(sx(use.min()), sy(a * use.min() + b), sx(use.max()), sy(a * use.max() + b), (220, 30, 30), dash=5)
    ideal = 1.0 / max(len(fr), 1)
    cv.line(ml, sy(ideal), ml + pw, sy(ideal), (128, 128, 128), dash=2)
    cv.axes(ml, mt, ml + pw, mt + ph)
    cv.text(ml, 8, f"layers using expert (of {nl}) vs token share  step {step}")
    cv.text(4, mt, f"{top:.4f}")
    for u in range(0, nl + 1, max(1, nl // 8)):
        cv.text(sx(u) - 3, mt + ph + 8, str(u))
    path = f"{prefix}_usage_vs_tokens.png"
    write_png(path, cv.img)
    return path
