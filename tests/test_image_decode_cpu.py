"""Damaged image files: the PNG / JPEG decoders of the vision path (models/vision.py, csrc/host/image.cc) answer a truncated or
corrupted file with ValueError or with an image, never with a crash (this file also runs under the sanitizers)."""
import io

import numpy as np
import pytest
import torch

from gemm_b200.models import vision

Image = pytest.importorskip("PIL.Image")


def _samples():
    g = np.random.default_rng(1)
    img = g.integers(0, 256, (37, 53, 3), dtype=np.uint8)
    img[:, :20] = 90
    out = []
    for fmt, kw in (("PNG", {}), ("JPEG", dict(quality=80, subsampling=2)), ("JPEG", dict(quality=90, subsampling=0, restart_marker_blocks=3))):
        buf = io.BytesIO()
        Image.fromarray(img).save(buf, fmt, **kw)
        out.append(buf.getvalue())
    buf = io.BytesIO()
    Image.fromarray(img).convert("P").save(buf, "PNG")
    out.append(buf.getvalue())
    return out


def test_damaged_files_never_crash():
    g = np.random.default_rng(2)
    n_err = n_ok = 0
    for data in _samples():
        assert vision.decode_image(data).shape == (37, 53, 3)
        trials = [data[:k] for k in range(0, len(data), max(1, len(data) // 60))]
        for _ in range(150):
            b = bytearray(data)
            for _ in range(int(g.integers(1, 6))):
                b[int(g.integers(2, len(b)))] = int(g.integers(0, 256))
            trials.append(bytes(b))
        for t in trials:
            try:
                img = vision.decode_image(t)
                assert img.dtype == torch.uint8 and img.dim() == 3 and img.shape[2] == 3
                n_ok += 1
            except ValueError:
                n_err += 1
    assert n_err > 50 and n_ok > 50
