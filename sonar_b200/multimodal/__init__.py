"""Multimodal inputs: image placeholders in the prompt and the tensors a vision encoder turns into embeddings.

A request carries ``multi_modal_data={"image": pixel_values | [pixel_values, …]}`` with already preprocessed
images (``[3, H, W]`` float tensors, resized and normalised the way the checkpoint's processor would do it) and
a prompt containing one image token per image.  The frontend replaces every image token by as many copies
as the encoder will produce embeddings (so that positions, KV blocks and the scheduler's token budget account
for them) and ships ``(start, count, "image", pixel_values)`` with the request; the worker runs the model's
encoder once per request and patches the resulting rows over the placeholder positions of the first layer's
input (``worker/model_runner.py`` ``_register_embeds``).  The prefix cache is salted with the image bytes.

Parity: ``aphrodite/multimodal/`` (processing: placeholder expansion, ``MultiModalKwargs``) and the
``get_multimodal_embeddings`` / ``get_input_embeddings`` pair of ``aphrodite/model_executor/models/llava.py``;
this build covers the LLaVA family (CLIP tower + MLP projector) and takes preprocessed pixel values only.
"""
from __future__ import annotations

import torch


def image_tokens_per_image(model_cfg) -> int:
    vc = model_cfg.get("vision_config") or {}
    grid = int(vc.get("image_size", 336)) // int(vc.get("patch_size", 14))
    n = grid * grid
    if model_cfg.get("vision_feature_select_strategy", "default") == "full":
        n += 1          # the class token stays
    return n


def expand_placeholders(model_cfg, tokenizer, prompt: dict) -> tuple[dict, list]:
    """→ (prompt dict with expanded ``prompt_token_ids``, ``[(start, count, kind, tensor)]``)."""
    mm = prompt["multi_modal_data"]
    unknown = set(mm) - {"image"}
    if unknown:
        raise ValueError(f"unsupported multimodal inputs {sorted(unknown)} (image only)")
    if model_cfg.get("vision_config") is None or model_cfg.get("image_token_index") is None:
        raise ValueError(f"model {model_cfg.model} takes no image inputs")
    images = mm["image"]
    images = list(images) if isinstance(images, (list, tuple)) else [images]
    images = [torch.as_tensor(im).float() for im in images]
    for im in images:
        if im.dim() == 4 and im.shape[0] == 1:
            im = im[0]
        if im.dim() != 3 or im.shape[0] != 3:
            raise ValueError(f"an image must be preprocessed pixel values [3, H, W], got {tuple(im.shape)}")
    images = [im[0] if im.dim() == 4 else im for im in images]
    ids = prompt.get("prompt_token_ids")
    if ids is None:
        if tokenizer is None:
            raise ValueError("text prompts with images need a tokenizer")
        ids = tokenizer.encode(prompt["prompt"])
    tok = int(model_cfg.get("image_token_index"))
    per = image_tokens_per_image(model_cfg)
    if sum(1 for t in ids if t == tok) != len(images):
        raise ValueError(f"the prompt has {sum(1 for t in ids if t == tok)} image tokens for {len(images)} images")
    out: list[int] = []
    items = []
    it = iter(images)
    for t in ids:
        if t == tok:
            items.append((len(out), per, "image", next(it).contiguous()))
            out.extend([tok] * per)
        else:
            out.append(int(t))
    new = {k: v for k, v in prompt.items() if k not in ("multi_modal_data", "prompt")}
    new["prompt_token_ids"] = out
    return new, items
