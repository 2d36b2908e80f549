"""Image transform programs and audio features."""
import io
import math
import struct
import wave

import numpy as np
import pytest
import torch

from onnx_genai_b200 import preprocess as pp


def test_image_program_resize_crop_normalize_and_layout():
    img = (np.arange(60 * 80 * 3) % 256).astype(np.uint8).reshape(60, 80, 3)
    prog = [{"op": "resize", "shortest_edge": 32}, {"op": "center_crop", "size": [32, 32]}, {"op": "rescale", "factor": 1 / 255},
            {"op": "normalize", "mean": [0.5, 0.5, 0.5], "std": [0.25, 0.25, 0.25]}]
    out = pp.run_image_program(img, prog)["pixel_values"]
    assert out.shape == (3, 32, 32) and out.dtype == torch.float32
    assert -2.01 <= float(out.min()) and float(out.max()) <= 2.01
    hwc = pp.run_image_program(img, prog + [{"op": "to_layout", "layout": "HWC"}])["pixel_values"]
    assert hwc.shape == (32, 32, 3) and torch.equal(hwc.permute(2, 0, 1), out)
    const = pp.run_image_program(np.full((10, 30, 3), 200, np.uint8), [{"op": "pad_to_square", "value": 0}, {"op": "resize", "size": [8, 8]}])
    assert const["pixel_values"].shape == (3, 8, 8)
    with pytest.raises(pp.PreprocessError, match="unknown image step"):
        pp.run_image_program(img, [{"op": "sharpen"}])
    with pytest.raises(pp.PreprocessError, match="channel statistics"):
        pp.run_image_program(img, [{"op": "normalize", "mean": [0.5], "std": [0.5]}])


def test_tiling_and_patch_packing():
    img = torch.rand(3, 100, 230)
    tiled = pp.run_image_program(img, [{"op": "tile", "size": [64, 64], "max_tiles": 6, "add_thumbnail": True}])
    rows, cols = tiled["grid"]
    assert rows * cols <= 6 and tiled["tiles"].shape == (rows * cols + 1, 3, 64, 64)
    packed = pp.run_image_program(img, [{"op": "patchify", "patch": 14, "merge": 2}])
    gh, gw = packed["grid"]
    assert gh % 2 == 0 and gw % 2 == 0 and packed["patches"].shape == (gh * gw, 3 * 14 * 14)
    # patch (0, 0) is the top-left 14x14 block of the (resized) image
    ref = packed["pixel_values"][:, :14, :14].reshape(-1)
    assert torch.allclose(packed["patches"][0], ref)
    # with merge = 2 the second packed patch is the right-hand neighbour, the third the one below
    assert torch.allclose(packed["patches"][1], packed["pixel_values"][:, :14, 14:28].reshape(-1))
    assert torch.allclose(packed["patches"][2], packed["pixel_values"][:, 14:28, :14].reshape(-1))


def _wav_bytes(x, rate, width=2, channels=1):
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(channels)
        w.setsampwidth(width)
        w.setframerate(rate)
        pcm = (np.clip(x, -1, 1) * 32767).astype("<i2")
        if channels == 2:
            pcm = np.stack([pcm, pcm], axis=1).reshape(-1)
        w.writeframes(pcm.tobytes())
    return buf.getvalue()


def test_wav_resample_and_log_mel():
    rate = 22050
    t = np.arange(rate) / rate
    tone = 0.5 * np.sin(2 * math.pi * 440.0 * t)
    x, r = pp.read_wav(_wav_bytes(tone, rate, channels=2))
    assert r == rate and len(x) == rate and abs(float(np.abs(x).max()) - 0.5) < 1e-3
    y = pp.resample(x, rate, 16000)
    assert abs(len(y) - 16000) <= 2
    spectrum = np.abs(np.fft.rfft(y[:16000]))
    assert abs(int(spectrum.argmax()) - 440) <= 2                      # the tone survives resampling at its frequency
    mel = pp.log_mel_spectrogram(y, 16000, pad_to_seconds=2.0)
    assert mel.shape == (80, 200) and torch.isfinite(mel).all()
    tone_frames, silent_frames = mel[:, :90], mel[:, 110:]
    assert float(tone_frames.max()) > float(silent_frames.max()) + 1.0  # energy where the tone is, floor where it is padded
    fb = pp.mel_filterbank(80, 400, 16000)
    assert fb.shape == (80, 201) and float(fb.min()) >= 0 and (fb.sum(1) > 0).all()
    with pytest.raises(pp.PreprocessError):
        pp.read_wav(b"RIFFxxxxWAVE")
    with pytest.raises(pp.PreprocessError):
        pp.read_wav(b"not a wave file at all")
    float_wav = b"RIFF" + struct.pack("<I", 36 + 8) + b"WAVE" + b"fmt " + struct.pack("<IHHIIHH", 16, 3, 1, 8000, 32000, 4, 32) + \
        b"data" + struct.pack("<I", 8) + struct.pack("<ff", 0.25, -0.5)
    xs, r8 = pp.read_wav(float_wav)
    assert r8 == 8000 and np.allclose(xs, [0.25, -0.5])


def test_declared_image_program_pixel_area_and_patch_layout():
    import io

    import numpy as np
    import torch
    from PIL import Image

    from onnx_genai_b200.preprocess import PreprocessError, pixel_area_size, run_declared_image_program

    # both sides multiples of 14, area inside the bounds when rounding allows, aspect kept
    assert pixel_area_size(8, 8, 224, 224, 14) == (28, 28)              # too small: scaled up, rounded up
    assert pixel_area_size(640, 480, 56 * 56, 28 * 28 * 16, 28) == (112, 84)
    assert pixel_area_size(29, 43, 100, 10 ** 6, 14) == (28, 42)        # already inside: just rounded (ties to even multiples)
    with pytest.raises(PreprocessError, match="aspect ratio"):
        pixel_area_size(2, 1000, 4, 10 ** 6, 2)
    spec = {"transforms": [{"op": "decode_rgb", "outputs": ["a"]},
                           {"op": "resize", "mode": "pixel_area", "interpolation": "bicubic", "min_pixels": 784, "max_pixels": 784, "size_multiple": 14,
                            "inputs": ["a"], "outputs": ["b"]},
                           {"op": "rescale", "scale": 1 / 255, "inputs": ["b"], "outputs": ["c"]},
                           {"op": "normalize", "mean": [0.5] * 3, "std": [0.5] * 3, "inputs": ["c"], "outputs": ["d"]},
                           {"op": "patchify", "patch_size": 14, "temporal_patch_size": 2, "merge_size": 1, "flatten": True, "inputs": ["d"], "outputs": ["e"]},
                           {"op": "emit_grid_coordinates", "inputs": ["e"], "outputs": ["g"]}],
            "outputs": [{"name": "image.pixel_values", "source": "e", "contract": {"shape": [4, 1176]}}, {"name": "image.grid_thw", "source": "g"}]}
    img = np.zeros((28, 28, 3), np.uint8)
    img[:14, 14:, 0] = 255                                               # the top-right patch is pure red
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    out = run_declared_image_program(buf.getvalue(), spec)
    assert out["image.grid_thw"].tolist() == [[1, 2, 2]] and out["image.pixel_values"].shape == (4, 1176)
    p = out["image.pixel_values"].reshape(4, 3, 2, 14, 14)               # patch, channel, temporal slot, y, x
    assert torch.allclose(p[1, 0], torch.ones(2, 14, 14)) and torch.allclose(p[1, 1], -torch.ones(2, 14, 14))
    assert torch.allclose(p[0], -torch.ones(3, 2, 14, 14)) and torch.equal(p[:, :, 0], p[:, :, 1])
    spec["outputs"][0]["contract"]["shape"] = [9, 1176]
    with pytest.raises(PreprocessError, match="contract says"):
        run_declared_image_program(buf.getvalue(), spec)
