"""Images of chat requests: fetch (``data:`` URLs; ``file://`` when a media root is configured), decode, and
preprocess the way a CLIP image processor does — resize the short side to the tower's input size (bicubic),
centre-crop, scale to [0, 1], normalise with the CLIP mean / standard deviation.

Parity: ``aphrodite/multimodal/media/image.py`` (``ImageMediaIO``: base64 / file loading) and the HF
``CLIPImageProcessor`` defaults that LLaVA checkpoints ship.
"""
from __future__ import annotations

import base64
import io
import os

import numpy as np
import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)
IMAGE_PLACEHOLDER = "<image>"


def load_image(url: str, allowed_local_path: str | None = None):
    from PIL import Image
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if ";base64" not in head:
            raise ValueError("data URLs must be base64 encoded")
        return Image.open(io.BytesIO(base64.b64decode(payload))).convert("RGB")
    if url.startswith("file://"):
        path = os.path.realpath(url[len("file://"):])
        root = os.path.realpath(allowed_local_path) if allowed_local_path else None
        if root is None or not path.startswith(root + os.sep):
            raise ValueError("local files are served only from the configured allowed_local_media_path")
        return Image.open(path).convert("RGB")
    raise ValueError("only data: and file:// image URLs are supported (this build makes no network requests)")


def preprocess_clip(img, size: int, mean=CLIP_MEAN, std=CLIP_STD) -> torch.Tensor:
    """PIL image → ``[3, size, size]`` float32."""
    from PIL import Image
    w, h = img.size
    scale = size / min(w, h)
    nw, nh = max(size, round(w * scale)), max(size, round(h * scale))
    img = img.resize((nw, nh), Image.BICUBIC)
    left, top = (nw - size) // 2, (nh - size) // 2
    img = img.crop((left, top, left + size, top + size))
    x = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
    return (x - torch.tensor(mean)[:, None, None]) / torch.tensor(std)[:, None, None]


def extract_chat_images(messages: list[dict], model_cfg, allowed_local_path: str | None = None
                        ) -> tuple[list[dict], list[torch.Tensor]]:
    """Replace every ``image_url`` content part by the text placeholder and return the preprocessed images in
    order of appearance."""
    size = int((model_cfg.get("vision_config") or {}).get("image_size", 336))
    images: list[torch.Tensor] = []
    out = []
    for m in messages:
        content = m.get("content")
        if isinstance(content, list):
            parts = []
            for p in content:
                if isinstance(p, dict) and p.get("type") in ("image_url", "input_image"):
                    ref = p.get("image_url")
                    url = ref.get("url") if isinstance(ref, dict) else ref
                    images.append(preprocess_clip(load_image(url, allowed_local_path), size))
                    parts.append({"type": "text", "text": IMAGE_PLACEHOLDER})
                else:
                    parts.append(p)
            m = {**m, "content": parts}
        out.append(m)
    return out, images


def encode_with_placeholders(tokenizer, text: str, image_token_id: int) -> list[int]:
    """Tokenise around the placeholders so that each becomes exactly one image token id, whatever the
    tokenizer would have made of the placeholder string."""
    pieces = text.split(IMAGE_PLACEHOLDER)
    ids: list[int] = []
    for i, piece in enumerate(pieces):
        if piece:
            ids.extend(tokenizer.encode(piece) if i == 0 else tokenizer.encode(piece, add_special_tokens=False))
        if i < len(pieces) - 1:
            ids.append(image_token_id)
    return ids
