"""Image and video preparation for vision-language prompts.

``process_image`` accepts what RL datasets store (a PIL image, ``{"bytes": ...}``, ``{"image": PIL | path}``, ``{"path": ...}``
or a path) and returns an RGB image whose sides are multiples of the vision tower's patch x merge size with the pixel count
inside ``[min_pixels, max_pixels]`` (aspect ratio kept as closely as the grid allows). ``process_video`` samples frames from
a list / array of frames (no container decoding here: decode with the library of your choice and pass the frames) and
resizes them the same way.

Parity target: ``verl/utils/dataset/vision_utils.py:22-106`` (``process_image``, ``process_video``).
"""

from __future__ import annotations

import math
from io import BytesIO
from typing import Any, Optional, Sequence

import numpy as np
import torch

__all__ = ["smart_resize", "process_image", "process_video"]


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """(height, width) rounded to multiples of ``factor`` with ``min_pixels <= h * w <= max_pixels`` where that is possible."""
    if min(height, width) <= 0:
        raise ValueError(f"empty image: {height} x {width}")
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio above 200: {height} x {width}")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _open(image: Any):
    from PIL import Image

    if isinstance(image, Image.Image):
        return image
    if isinstance(image, str):
        return Image.open(image)
    if isinstance(image, bytes):
        return Image.open(BytesIO(image))
    if isinstance(image, np.ndarray):
        return Image.fromarray(image.astype(np.uint8))
    if isinstance(image, torch.Tensor):      # [C, H, W] or [H, W, C], 0..255
        a = image.detach().cpu()
        if a.dim() == 3 and a.shape[0] in (1, 3) and a.shape[-1] not in (1, 3):
            a = a.permute(1, 2, 0)
        return Image.fromarray(a.to(torch.uint8).numpy().squeeze())
    if isinstance(image, dict):
        if "bytes" in image and image["bytes"] is not None:
            assert image.get("image") is None, "an image record holds either `bytes` or `image`, not both"
            return Image.open(BytesIO(image["bytes"]))
        for key in ("image", "path"):
            if image.get(key) is not None:
                return _open(image[key])
    raise TypeError(f"cannot read an image from {type(image).__name__}")


def process_image(image: Any, image_patch_size: int = 14, merge_size: int = 2, min_pixels: Optional[int] = None,
                  max_pixels: Optional[int] = None):
    """RGB PIL image on the vision tower's grid. Per-record ``min_pixels`` / ``max_pixels`` (dict records) win over the
    arguments; without any limit the image is only rounded to the grid."""
    from PIL import Image

    rec = image if isinstance(image, dict) else {}
    img = _open(image).convert("RGB")
    factor = image_patch_size * merge_size
    lo = rec.get("min_pixels", min_pixels)
    hi = rec.get("max_pixels", max_pixels)
    h, w = smart_resize(img.height, img.width, factor, lo if lo is not None else factor * factor,
                        hi if hi is not None else max(img.height * img.width, factor * factor))
    if (h, w) != (img.height, img.width):
        img = img.resize((w, h), Image.BICUBIC)
    return img


def process_video(video: Any, image_patch_size: int = 14, merge_size: int = 2, nframes: Optional[int] = None, fps: Optional[float] = None,
                  source_fps: float = 30.0, fps_min_frames: int = 4, fps_max_frames: int = 768, temporal_patch: int = 2,
                  min_pixels: Optional[int] = None, max_pixels: Optional[int] = None) -> torch.Tensor:
    """``[frames, 3, H, W]`` uint8 tensor. ``video``: a sequence / array of frames, or a record ``{"video": frames, "fps": ...,
    "nframes": ..., "min_pixels": ..., "max_pixels": ...}``. Exactly one of ``nframes`` / ``fps`` picks the sampling (default:
    2 frames per second of a 30 fps source); the count is rounded to a multiple of the temporal patch size."""
    rec = video if isinstance(video, dict) else {}
    frames = rec.get("video", video) if rec else video
    if isinstance(frames, (str, bytes)):
        raise NotImplementedError("container decoding is not part of this module: pass decoded frames")
    nframes = rec.get("nframes", nframes)
    fps = rec.get("fps", fps)
    assert nframes is None or fps is None, "give nframes or fps, not both"
    total = len(frames)
    if nframes is None:
        want = total / float(rec.get("source_fps", source_fps)) * float(fps if fps is not None else 2.0)
        nframes = min(max(want, fps_min_frames), min(fps_max_frames, total))
    n = int(max(temporal_patch, math.floor(min(nframes, total) / temporal_patch) * temporal_patch))
    idx = torch.linspace(0, total - 1, n).round().long().tolist()
    out = []
    for i in idx:
        img = process_image(frames[i], image_patch_size, merge_size, rec.get("min_pixels", min_pixels), rec.get("max_pixels", max_pixels))
        out.append(torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1))
    return torch.stack(out)
