"""`transcribe` subcommand: segmentation of files and live streams, the three transcript formats, argument errors."""
import argparse
import io
import json
import struct

import numpy as np
import pytest

from onnx_genai_b200 import cli
from onnx_genai_b200.preprocess import StreamSegmenter, write_wav


class CountingTranscriber:
    """Stands in for a speech model: reports how many samples it was given and at what rate it wants them."""
    sample_rate = 16000
    window_seconds = 2.0

    def __init__(self):
        self.calls = []

    def transcribe(self, samples, language=None):
        self.calls.append((len(samples), language))
        return "" if np.abs(samples).max() < 1e-3 else f"{len(samples)} samples"


def _args(**kw):
    base = dict(model="unused", audio=[], language="", format="text", segment_seconds=0.0, silence_seconds=0.5,
                silence_threshold=0.01, min_segment_seconds=0.1, sample_rate=16000, channels=1, device="cpu")
    base.update(kw)
    return argparse.Namespace(**base)


def _speech(rate, seconds, amp=0.5):
    t = np.arange(int(rate * seconds)) / rate
    return (amp * np.sin(2 * np.pi * 220 * t)).astype(np.float32)


def test_segmenter_cuts_on_silence_and_on_the_window():
    rate = 1000
    seg = StreamSegmenter(rate, max_seconds=1.0, silence_seconds=0.1, silence_rms=0.01, min_seconds=0.05)
    x = np.concatenate([_speech(rate, 0.4), np.zeros(300, np.float32), _speech(rate, 1.7), np.zeros(200, np.float32),
                        _speech(rate, 0.02), np.zeros(200, np.float32), _speech(rate, 0.3)])
    got = []
    for i in range(0, len(x), 137):                       # arrives in arbitrary chunks
        got += seg.push(x[i:i + 137])
    last = seg.flush()
    if last is not None:
        got.append(last)
    starts = [s for _, s in got]
    lens = [len(a) for a, _ in got]
    # 0.4 s burst, then the 1.7 s burst split by the window (1.0 + 0.7), the 20 ms click dropped, the final 0.3 s burst
    assert starts[0] == 0 and abs(lens[0] - 400) <= 1
    assert starts[1] in (700, 701) and lens[1] == 1000 and lens[2] in range(695, 705)
    assert len(got) == 4 and abs(lens[3] - 300) <= 1 and starts[3] >= 2800


def test_transcribe_files_in_every_format(tmp_path):
    rate = 16000
    wav = tmp_path / "a.wav"
    wav.write_bytes(write_wav(np.concatenate([_speech(rate, 1.0), np.zeros(rate, np.float32), _speech(rate, 0.5)]), rate))
    for fmt in ("text", "json", "srt"):
        tr, out = CountingTranscriber(), io.StringIO()
        rc = cli.cmd_transcribe(_args(audio=[str(wav)], format=fmt, language="en"), cli.Profiler(False), transcriber=tr, out=out)
        assert rc == 0 and len(tr.calls) == 2 and tr.calls[0][1] == "en"
        text = out.getvalue()
        near = lambda line, want: abs(int(line.split()[0]) - want) <= 2      # a burst may begin or end on a zero crossing
        if fmt == "text":
            a, b = text.splitlines()
            assert near(a, 16000) and near(b, 8000)
        elif fmt == "json":
            rows = [json.loads(line) for line in text.splitlines()]
            assert [r["index"] for r in rows] == [0, 1] and rows[0]["start"] == 0.0 and abs(rows[0]["end"] - 1.0) < 1e-3
            assert abs(rows[1]["start"] - 2.0) < 2e-3 and abs(rows[1]["end"] - 2.5) < 2e-3
        else:
            lines = text.split("\n")
            assert lines[0] == "1" and lines[1] == "00:00:00,000 --> 00:00:01,000" and near(lines[2], 16000) and lines[3] == ""
            assert lines[4] == "2" and lines[5] == "00:00:02,000 --> 00:00:02,500" and near(lines[6], 8000)
    assert cli.srt_timestamp(3725.0415) == "01:02:05,042"


def test_transcribe_a_live_stream_raw_and_with_a_wav_header():
    rate = 8000
    x = np.concatenate([_speech(rate, 0.5), np.zeros(rate, np.float32), _speech(rate, 0.25)])
    stereo = np.stack([x, x], axis=1).reshape(-1)
    pcm = (np.clip(stereo, -1, 1) * 32767).astype("<i2").tobytes()
    tr, out = CountingTranscriber(), io.StringIO()
    rc = cli.cmd_transcribe(_args(sample_rate=rate, channels=2), cli.Profiler(False), transcriber=tr, stdin=io.BytesIO(pcm), out=out)
    assert rc == 0
    assert len(tr.calls) == 2 and abs(tr.calls[0][0] - 8000) <= 4 and abs(tr.calls[1][0] - 4000) <= 4   # resampled to the model's 16 kHz
    # the same samples behind a WAV header whose data chunk claims no length (a pipe): rate and channels come from the header
    header = (b"RIFF" + struct.pack("<I", 0xFFFFFFFF) + b"WAVE" + b"fmt " + struct.pack("<IHHIIHH", 16, 1, 2, rate, rate * 4, 4, 16)
              + b"data" + struct.pack("<I", 0xFFFFFFFF))
    tr2, out2 = CountingTranscriber(), io.StringIO()
    rc = cli.cmd_transcribe(_args(sample_rate=44100, channels=1), cli.Profiler(False), transcriber=tr2, stdin=io.BytesIO(header + pcm), out=out2)
    assert rc == 0 and out2.getvalue() == out.getvalue()


def test_transcribe_rejects_segments_longer_than_the_window_and_bad_files(tmp_path, capsys):
    tr = CountingTranscriber()
    assert cli.cmd_transcribe(_args(audio=["-"], segment_seconds=5.0), cli.Profiler(False), transcriber=tr, stdin=io.BytesIO(b"")) == 2
    assert "holds at most 2.00s" in capsys.readouterr().err
    bad = tmp_path / "x.wav"
    bad.write_bytes(b"not audio")
    assert cli.cmd_transcribe(_args(audio=[str(bad)]), cli.Profiler(False), transcriber=tr) == 2
    assert "could not be decoded" in capsys.readouterr().err
    assert cli.cmd_transcribe(_args(audio=[str(tmp_path / "missing.wav")]), cli.Profiler(False), transcriber=tr) == 2


def test_transcribe_is_a_subcommand():
    with pytest.raises(SystemExit):
        cli.main(["transcribe", "--help"])
