"""Declared input preprocessing for multimodal front ends: image transform programs and audio features.

The inference-metadata standard lets a model declare how raw inputs become tensors; the reference executes those
declarations in its preprocess crate (crates/onnx-genai-preprocess/src/image/program.rs: resize / crop / pad /
rescale / normalize / layout / tile steps; src/image/packed.rs: patch packing for NaViT-style encoders;
src/audio.rs: WAV decoding, resampling and log-mel features).  This module runs the same declarations with
torch, on the CPU or on the GPU the tensors live on.  It is not on the text-generation path: the decoder-only
configurations never call it.

An image program is a list of steps, each a dict with an ``op`` key:

    {"op": "resize", "size": [h, w] | "shortest_edge": n | "longest_edge": n, "interpolation": "bilinear|bicubic|nearest"}
    {"op": "center_crop", "size": [h, w]}
    {"op": "pad_to_square", "value": 0}          {"op": "pad", "size": [h, w], "value": 0}
    {"op": "rescale", "factor": 1/255}           {"op": "normalize", "mean": [...], "std": [...]}
    {"op": "to_layout", "layout": "CHW" | "HWC"}
    {"op": "tile", "size": [h, w], "max_tiles": n, "add_thumbnail": true}
    {"op": "patchify", "patch": p, "merge": m}    # -> [num_patches, C*p*p] plus the (rows, cols) grid

Audio: :func:`read_wav`, :func:`resample`, :func:`log_mel_spectrogram` (Whisper-style 80/128-bin features).
"""
from __future__ import annotations

import math
import struct

import numpy as np
import torch
import torch.nn.functional as F

_INTERP = {"bilinear": "bilinear", "bicubic": "bicubic", "nearest": "nearest"}


class PreprocessError(ValueError):
    pass


def _as_chw_float(image) -> torch.Tensor:
    """uint8/float HWC or CHW array or tensor -> float32 CHW tensor (values unchanged)."""
    t = torch.as_tensor(np.asarray(image)) if not isinstance(image, torch.Tensor) else image
    if t.dim() == 2:
        t = t[..., None]
    if t.dim() != 3:
        raise PreprocessError(f"an image must have 2 or 3 dimensions, got shape {tuple(t.shape)}")
    if t.shape[-1] in (1, 3, 4) and t.shape[0] not in (1, 3, 4):
        t = t.permute(2, 0, 1)
    elif t.shape[0] not in (1, 3, 4):
        raise PreprocessError(f"cannot tell the channel axis of an image of shape {tuple(t.shape)}")
    return t.float()


def _resize(img, h, w, interpolation):
    mode = _INTERP.get(interpolation)
    if mode is None:
        raise PreprocessError(f"unknown interpolation {interpolation!r}; use bilinear, bicubic or nearest")
    kw = {} if mode == "nearest" else {"align_corners": False, "antialias": True}
    return F.interpolate(img[None], size=(int(h), int(w)), mode=mode, **kw)[0]


def run_image_program(image, program) -> dict:
    """Apply ``program`` to one image.  Returns ``{"pixel_values": tensor, ...}`` plus ``tiles`` / ``grid`` entries
    when the program tiles or patchifies."""
    img = _as_chw_float(image)
    out: dict = {}
    layout = "CHW"
    for step in program:
        op = step.get("op")
        if op == "resize":
            _, h, w = img.shape
            if "size" in step:
                nh, nw = step["size"]
            elif "shortest_edge" in step:
                s = step["shortest_edge"] / min(h, w)
                nh, nw = round(h * s), round(w * s)
            elif "longest_edge" in step:
                s = step["longest_edge"] / max(h, w)
                nh, nw = round(h * s), round(w * s)
            else:
                raise PreprocessError("resize needs size, shortest_edge or longest_edge")
            img = _resize(img, max(1, nh), max(1, nw), step.get("interpolation", "bilinear"))
        elif op == "center_crop":
            ch, cw = step["size"]
            _, h, w = img.shape
            if ch > h or cw > w:
                img = F.pad(img, (0, max(0, cw - w), 0, max(0, ch - h)))
                _, h, w = img.shape
            top, left = (h - ch) // 2, (w - cw) // 2
            img = img[:, top:top + ch, left:left + cw]
        elif op == "pad_to_square":
            _, h, w = img.shape
            side = max(h, w)
            img = F.pad(img, ((side - w) // 2, side - w - (side - w) // 2, (side - h) // 2, side - h - (side - h) // 2),
                        value=float(step.get("value", 0)))
        elif op == "pad":
            ph, pw = step["size"]
            _, h, w = img.shape
            if ph < h or pw < w:
                raise PreprocessError(f"pad target {ph}x{pw} is smaller than the image {h}x{w}")
            img = F.pad(img, (0, pw - w, 0, ph - h), value=float(step.get("value", 0)))
        elif op == "rescale":
            img = img * float(step["factor"])
        elif op == "normalize":
            mean = torch.tensor(step["mean"], dtype=img.dtype, device=img.device)[:, None, None]
            std = torch.tensor(step["std"], dtype=img.dtype, device=img.device)[:, None, None]
            if mean.shape[0] != img.shape[0]:
                raise PreprocessError(f"normalize has {mean.shape[0]} channel statistics for {img.shape[0]} channels")
            img = (img - mean) / std
        elif op == "to_layout":
            layout = step["layout"].upper()
            if layout not in ("CHW", "HWC"):
                raise PreprocessError(f"unknown layout {step['layout']!r}")
        elif op == "tile":
            th, tw = step["size"]
            _, h, w = img.shape
            rows, cols = max(1, math.ceil(h / th)), max(1, math.ceil(w / tw))
            max_tiles = int(step.get("max_tiles", rows * cols))
            while rows * cols > max_tiles:          # shrink the grid along its longer side until it fits
                if rows >= cols and rows > 1:
                    rows -= 1
                elif cols > 1:
                    cols -= 1
                else:
                    break
            canvas = _resize(img, rows * th, cols * tw, step.get("interpolation", "bilinear"))
            tiles = canvas.unfold(1, th, th).unfold(2, tw, tw).permute(1, 2, 0, 3, 4).reshape(rows * cols, img.shape[0], th, tw)
            if step.get("add_thumbnail", False) and rows * cols > 1:
                tiles = torch.cat([tiles, _resize(img, th, tw, step.get("interpolation", "bilinear"))[None]])
            out["tiles"] = tiles
            out["grid"] = (rows, cols)
        elif op == "patchify":
            p = int(step["patch"])
            merge = int(step.get("merge", 1))
            _, h, w = img.shape
            unit = p * merge
            nh, nw = max(unit, round(h / unit) * unit), max(unit, round(w / unit) * unit)
            if (nh, nw) != (h, w):
                img = _resize(img, nh, nw, step.get("interpolation", "bicubic"))
            c = img.shape[0]
            gh, gw = nh // p, nw // p
            patches = img.reshape(c, gh, p, gw, p).permute(1, 3, 0, 2, 4)          # [gh, gw, C, p, p]
            if merge > 1:      # keep merge x merge neighbours adjacent, as window-merging encoders expect
                patches = patches.reshape(gh // merge, merge, gw // merge, merge, c, p, p).permute(0, 2, 1, 3, 4, 5, 6)
            out["patches"] = patches.reshape(gh * gw, c * p * p)
            out["grid"] = (gh, gw)
        else:
            raise PreprocessError(f"unknown image step {op!r}; supported: resize, center_crop, pad_to_square, pad, rescale, "
                                  "normalize, to_layout, tile, patchify")
    out["pixel_values"] = img.permute(1, 2, 0) if layout == "HWC" else img
    return out


# ---------------------------------------------------------------------------------------------
# audio
# ---------------------------------------------------------------------------------------------
def read_wav(data: bytes):
    """(samples float32 mono in [-1, 1], sample_rate) from RIFF/WAVE bytes: PCM 8/16/24/32-bit or IEEE float."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise PreprocessError("not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        tag, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        body = data[pos + 8:pos + 8 + size]
        if tag == b"fmt ":
            fmt = struct.unpack("<HHIIHH", body[:16])
        elif tag == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise PreprocessError("WAVE file lacks a fmt or data chunk")
    code, channels, rate, _, _, bits = fmt
    if code == 1 and bits == 16:
        x = np.frombuffer(pcm, dtype="<i2").astype(np.float32) / 32768.0
    elif code == 1 and bits == 8:
        x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif code == 1 and bits == 32:
        x = np.frombuffer(pcm, dtype="<i4").astype(np.float32) / 2147483648.0
    elif code == 1 and bits == 24:
        b = np.frombuffer(pcm[: len(pcm) // 3 * 3], dtype=np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / 8388608.0
    elif code == 3 and bits == 32:
        x = np.frombuffer(pcm, dtype="<f4").astype(np.float32)
    else:
        raise PreprocessError(f"unsupported WAVE encoding (format {code}, {bits} bits); use PCM 8/16/24/32 or float32")
    if channels > 1:
        x = x[: len(x) // channels * channels].reshape(-1, channels).mean(axis=1)
    return x.astype(np.float32), int(rate)


def write_wav(samples, sample_rate: int) -> bytes:
    """RIFF/WAVE bytes, 16-bit little-endian PCM.  ``samples``: [n] mono or [channels, n], floats in [-1, 1] (clipped)."""
    x = np.asarray(samples, dtype=np.float32)
    if x.ndim == 1:
        x = x[None]
    if x.ndim != 2 or x.shape[0] > 8:
        raise PreprocessError(f"write_wav wants [n] or [channels, n] with at most 8 channels, got {list(x.shape)}")
    channels, n = x.shape
    pcm = (np.clip(x, -1.0, 1.0) * 32767.0).round().astype("<i2").T.reshape(-1).tobytes()       # interleaved frames
    fmt = struct.pack("<HHIIHH", 1, channels, int(sample_rate), int(sample_rate) * channels * 2, channels * 2, 16)
    return b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVE" + b"fmt " + struct.pack("<I", 16) + fmt + b"data" + struct.pack("<I", len(pcm)) + pcm


def resample(samples, src_rate: int, dst_rate: int, taps: int = 32) -> np.ndarray:
    """Band-limited (Hann-windowed sinc) resampling: each output sample is a weighted sum of the 2*taps+1 input
    samples around its position, with the cut-off at the lower of the two Nyquist rates."""
    x = np.asarray(samples, dtype=np.float32)
    if src_rate == dst_rate or len(x) == 0:
        return x
    ratio = dst_rate / src_rate
    cutoff = min(1.0, ratio)                                   # relative to the source Nyquist rate
    width = taps / cutoff                                       # half-width of the kernel in source samples
    n_out = int(math.floor(len(x) * ratio))
    pos = torch.arange(n_out, dtype=torch.float64) / ratio      # output positions on the source grid
    base = torch.floor(pos).long()
    offs = torch.arange(-int(math.ceil(width)), int(math.ceil(width)) + 1)
    idx = base[:, None] + offs[None, :]
    d = pos[:, None] - idx.double()
    w = cutoff * torch.sinc(cutoff * d) * (0.5 + 0.5 * torch.cos(math.pi * d / width)).clamp_min(0.0) * (d.abs() <= width)
    xt = torch.as_tensor(x, dtype=torch.float64)
    gathered = xt[idx.clamp(0, len(x) - 1)] * ((idx >= 0) & (idx < len(x)))
    return (gathered * w).sum(1).float().numpy()


class StreamSegmenter:
    """Cuts a growing waveform into transcribable segments, incrementally.

    A speech encoder takes a bounded window, so a long recording -- or a live stream -- is split before it is
    transcribed: at a run of silence when there is one (words stay whole), at the window bound otherwise.  Feed
    whatever arrives to :meth:`push`; it returns the segments that became final as ``(samples, start_sample)``;
    :meth:`flush` returns the trailing partial segment once the input ends.  Nothing beyond the current segment is
    buffered.  Behaviour follows the reference's segmenter (crates/onnx-genai-preprocess/src/audio.rs:225-382):
    a sample is silent when its square is at most ``silence_rms**2``; ``silence_seconds`` of consecutive silence end
    a segment and are dropped, as is the rest of the gap; a voiced burst shorter than ``min_seconds`` between two
    silences is discarded; a cut forced by the window keeps everything, silence included."""

    def __init__(self, sample_rate: int, max_seconds: float, silence_seconds: float = 0.5, silence_rms: float = 0.01,
                 min_seconds: float = 0.1):
        if sample_rate <= 0:
            raise PreprocessError("the sample rate must be positive")
        n = lambda sec: int(round(max(0.0, float(sec)) * sample_rate))
        self.max_samples = n(max_seconds)
        if self.max_samples == 0:
            raise PreprocessError("the maximum segment length rounds to zero samples")
        self.silence_samples = n(silence_seconds)
        self.threshold = max(0.0, float(silence_rms)) ** 2
        self.min_samples = min(n(min_seconds), self.max_samples)
        self.pending: list = []          # chunks of the current segment
        self.pending_len = 0
        self.pending_start = 0           # stream position of the first pending sample
        self.trailing_silence = 0
        self.in_gap = False

    def _take(self, forced: bool):
        voiced = self.pending_len - self.trailing_silence
        keep = self.pending_len if forced else voiced
        total = self.pending_len
        buf = np.concatenate(self.pending) if self.pending else np.zeros(0, np.float32)
        self.pending, self.pending_len, self.trailing_silence = [], 0, 0
        start = self.pending_start
        self.pending_start += total
        if keep == 0 or (not forced and keep < self.min_samples):
            return None
        return buf[:keep].astype(np.float32), start

    def push(self, samples):
        x = np.asarray(samples, dtype=np.float32).reshape(-1)
        silent = x * x <= self.threshold
        out, i, n = [], 0, len(x)
        while i < n:
            if self.in_gap:
                nz = np.flatnonzero(~silent[i:])
                if len(nz) == 0:                       # the rest of this chunk is still the gap: drop it
                    self.pending_start += n - i
                    break
                self.pending_start += int(nz[0])
                i += int(nz[0])
                self.in_gap = False
            # how far can the current segment grow before one of the two cuts fires?
            room = self.max_samples - self.pending_len
            j_end = min(n, i + room)
            cut = None
            if self.silence_samples > 0:
                # position (exclusive) at which the run of trailing silence reaches silence_samples
                run = self.trailing_silence
                seg = silent[i:j_end]
                if seg.all():
                    if run + len(seg) >= self.silence_samples:
                        cut = i + (self.silence_samples - run)
                else:
                    # runs inside the chunk: scan for the first run (continuing `run`) that is long enough
                    idx = np.flatnonzero(~seg)
                    if run + int(idx[0]) >= self.silence_samples:
                        cut = i + (self.silence_samples - run)
                    else:
                        gaps = np.diff(np.concatenate([idx, [len(seg)]])) - 1      # silent samples after each voiced one
                        hit = np.flatnonzero(gaps >= self.silence_samples)
                        if len(hit):
                            cut = i + int(idx[hit[0]]) + 1 + self.silence_samples
            stop = cut if cut is not None else j_end
            piece = x[i:stop]
            if len(piece):
                self.pending.append(piece)
                self.pending_len += len(piece)
                sil = silent[i:stop]
                if sil.all():
                    self.trailing_silence += len(piece)
                else:
                    self.trailing_silence = len(piece) - 1 - int(np.flatnonzero(~sil)[-1])
            i = stop
            hit_window = self.pending_len >= self.max_samples
            hit_silence = self.silence_samples > 0 and self.trailing_silence >= self.silence_samples
            if hit_window or hit_silence:
                seg_out = self._take(hit_window)
                if seg_out is not None:
                    out.append(seg_out)
                self.in_gap = self.silence_samples > 0 and self.pending_len == 0
        return out

    def flush(self):
        return self._take(False)


def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int) -> torch.Tensor:
    """Slaney-style triangular mel filters [n_mels, n_fft//2 + 1] (the scale Whisper's features use)."""
    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        return np.where(f < 1000.0, f / (200.0 / 3), 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0))

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        return np.where(m < 15.0, m * (200.0 / 3), 1000.0 * np.exp((m - 15.0) * (np.log(6.4) / 27.0)))

    freqs = np.linspace(0, sample_rate / 2, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(sample_rate / 2), n_mels + 2))
    fb = np.zeros((n_mels, len(freqs)))
    for i in range(n_mels):
        lo, mid, hi = pts[i], pts[i + 1], pts[i + 2]
        up = (freqs - lo) / max(mid - lo, 1e-10)
        dn = (hi - freqs) / max(hi - mid, 1e-10)
        fb[i] = np.maximum(0.0, np.minimum(up, dn)) * (2.0 / (hi - lo))
    return torch.tensor(fb, dtype=torch.float32)


def log_mel_spectrogram(samples, sample_rate: int = 16000, n_fft: int = 400, hop: int = 160, n_mels: int = 80,
                        pad_to_seconds: float | None = 30.0, device="cpu") -> torch.Tensor:
    """[n_mels, frames] log10-mel features, clamped to 8 dB below the peak and scaled to roughly [-1, 1]."""
    x = torch.as_tensor(np.asarray(samples, dtype=np.float32), device=device)
    if pad_to_seconds:
        want = int(pad_to_seconds * sample_rate)
        x = x[:want] if len(x) >= want else F.pad(x, (0, want - len(x)))
    window = torch.hann_window(n_fft, device=x.device)
    spec = torch.stft(x, n_fft, hop, window=window, return_complex=True)[:, :-1].abs() ** 2
    mel = mel_filterbank(n_mels, n_fft, sample_rate).to(x.device) @ spec
    log = torch.clamp(mel, min=1e-10).log10()
    log = torch.maximum(log, log.max() - 8.0)
    return (log + 4.0) / 4.0


# ---------------------------------------------------------------------------------------------
# declared transform programs (the ``preprocessing.image`` block of the inference metadata)
# ---------------------------------------------------------------------------------------------
def _round_half_even_to(value: int, multiple: int) -> int:
    q, r = divmod(value, multiple)
    if 2 * r > multiple or (2 * r == multiple and q % 2 == 1):
        q += 1
    return q * multiple


def pixel_area_size(width: int, height: int, min_pixels: int, max_pixels: int, multiple: int):
    """Target (width, height) of an area-bounded resize: both sides are multiples of ``multiple`` and the area lies in
    [min_pixels, max_pixels] as far as rounding allows, keeping the aspect ratio -- the dynamic-resolution rule of
    patch-based vision encoders (crates/onnx-genai-preprocess/src/image/transform.rs:42-70)."""
    if not (0 < min_pixels <= max_pixels and multiple > 0):
        raise PreprocessError("pixel_area resize needs 0 < min_pixels <= max_pixels and size_multiple > 0")
    if max(width, height) / max(1, min(width, height)) > 200:
        raise PreprocessError(f"pixel_area resize needs an aspect ratio of at most 200, got {width}x{height}")
    w, h = _round_half_even_to(width, multiple), _round_half_even_to(height, multiple)
    if w * h > max_pixels:
        beta = math.sqrt(width * height / max_pixels)
        h = max(1, math.floor(height / beta / multiple)) * multiple
        w = max(1, math.floor(width / beta / multiple)) * multiple
    elif w * h < min_pixels:
        beta = math.sqrt(min_pixels / (width * height))
        h = max(1, math.ceil(height * beta / multiple)) * multiple
        w = max(1, math.ceil(width * beta / multiple)) * multiple
    return w, h


def decode_rgb(encoded) -> torch.Tensor:
    """Encoded image bytes (PNG, JPEG, ...) -> uint8-valued float tensor [3, H, W]."""
    import io

    from PIL import Image

    data = bytes(encoded.cpu().numpy().astype(np.uint8).tobytes()) if isinstance(encoded, torch.Tensor) else bytes(np.asarray(encoded, dtype=np.uint8).tobytes()) \
        if not isinstance(encoded, (bytes, bytearray)) else bytes(encoded)
    try:
        img = Image.open(io.BytesIO(data)).convert("RGB")
    except Exception as e:
        raise PreprocessError(f"cannot decode the image ({len(data)} bytes): {e}") from e
    return torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float()


def run_declared_image_program(image, spec: dict) -> dict:
    """Run the ``transforms`` of a ``preprocessing.image`` block on one image (encoded bytes, or an array [H, W, 3] /
    [3, H, W]) and return its declared ``outputs`` by name.  Transforms name their inputs and outputs; covered operators:
    ``decode_rgb``, ``resize`` (modes ``stretch`` and ``pixel_area``), ``rescale``, ``normalize``, ``patchify`` (with temporal
    replication and merge windows) and ``emit_grid_coordinates``."""
    values: dict = {}
    source, last = image, None
    for i, tr in enumerate(spec.get("transforms") or []):
        op = tr.get("op")
        ins = [values[n] for n in tr.get("inputs") or []]
        x = ins[0] if ins else None
        if op == "decode_rgb":
            y = decode_rgb(source) if isinstance(source, (bytes, bytearray)) or (hasattr(source, "ndim") and source.ndim == 1) else _as_chw_float(source)
        elif op == "resize":
            _, h, w = x.shape
            mode = tr.get("mode", "stretch")
            if mode == "pixel_area":
                nw, nh = pixel_area_size(w, h, int(tr["min_pixels"]), int(tr["max_pixels"]), int(tr["size_multiple"]))
            elif mode == "stretch":
                nh, nw = int(tr["height"]), int(tr["width"])
            else:
                raise PreprocessError(f"transform {i}: resize mode {mode!r} is not covered (stretch, pixel_area)")
            y = _resize(x, nh, nw, tr.get("interpolation", "bilinear"))
        elif op == "rescale":
            y = x * float(tr["scale"])
        elif op == "normalize":
            mean = torch.tensor(tr["mean"], dtype=x.dtype)[:, None, None]
            std = torch.tensor(tr["std"], dtype=x.dtype)[:, None, None]
            y = (x - mean) / std
        elif op == "patchify":
            p, t, m = int(tr["patch_size"]), int(tr.get("temporal_patch_size", 1)), int(tr.get("merge_size", 1))
            c, h, w = x.shape
            if h % (p * m) or w % (p * m):
                raise PreprocessError(f"transform {i}: a {h}x{w} image does not split into {p}-pixel patches in {m}x{m} windows; resize first")
            gh, gw = h // p, w // p
            frames = x[None].expand(t, c, h, w)                          # a still image fills every temporal slot
            v = frames.reshape(1, t, c, gh // m, m, p, gw // m, m, p).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
            y = v.reshape(gh * gw, c * t * p * p) if tr.get("flatten", True) else v.reshape(gh * gw, c, t, p, p)
            values["__grid__"] = torch.tensor([[1, gh, gw]], dtype=torch.int64)
        elif op == "emit_grid_coordinates":
            if "__grid__" not in values:
                raise PreprocessError(f"transform {i}: emit_grid_coordinates needs a patchify step before it")
            y = values["__grid__"]
        else:
            raise PreprocessError(f"transform {i}: unknown operator {op!r}; covered: decode_rgb, resize, rescale, normalize, patchify, "
                                  "emit_grid_coordinates")
        for name in tr.get("outputs") or []:
            values[name] = y
        last = y
    out = {}
    for o in spec.get("outputs") or []:
        if o.get("source") not in values:
            raise PreprocessError(f"output {o.get('name')!r} reads {o.get('source')!r}, which no transform produced")
        v = values[o["source"]]
        want = (o.get("contract") or {}).get("shape")
        if want and all(isinstance(d, int) for d in want) and list(v.shape) != list(want):
            raise PreprocessError(f"output {o['name']!r} has shape {list(v.shape)} but its contract says {want}")
        out[o["name"]] = v
    if not out and last is not None:
        out["pixel_values"] = last
    return out


def image_preprocess_adapter(spec: dict, input_port: str = "encoded"):
    """A workflow component for the ``onnx-genai.image-preprocess`` adapter: encoded bytes in, the program's outputs out
    (port names are the output names without their ``image.`` prefix)."""
    def component(ports: dict) -> dict:
        res = run_declared_image_program(ports[input_port], spec)
        return {name.split(".", 1)[-1]: v for name, v in res.items()}

    return component
