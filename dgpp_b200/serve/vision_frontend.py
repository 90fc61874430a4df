"""Vision frontend of the chat endpoint: image content parts -> visual tokens in the prompt + embedding rows.

The chat template still renders roles, tools and reasoning from the checkpoint's own template; each `image_url` part
of a message is replaced, before rendering, by a sentinel that survives the template untouched.  The rendered text is
then cut at the sentinels, the text pieces are tokenised on their own, and every image becomes
`[start id] + one id per visual token + [end id]`.  Towards the scheduler the per-token ids are pseudo ids >= vocab
derived from a hash of the image canvas (two different images never share a prefix-cache block); the engine maps them
to the family's pad id and overwrites the rows with the vision tower's output (`EmbedSplice`).
(reference counterparts: src/serve/vision_frontend.cpp prepare_chat, glm_vision_frontend.hpp / qwen_vision_frontend.hpp
 specs, docs/vision.md.)
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

import torch

from .image_inputs import ImageInputError, ImagePreprocess, prepare_image

SENTINEL = "\ufffc"     # OBJECT REPLACEMENT CHARACTER; stripped from user text before it brackets an image index
MAX_IMAGES_PER_REQUEST = 16


@dataclass
class VisionSpec:
    start_id: int
    pad_id: int
    end_id: int
    preprocess: ImagePreprocess = field(default_factory=ImagePreprocess)


def _remix(digest48: int, j: int) -> int:
    """30 bits of splitmix64(digest + golden * (j + 1))."""
    x = (digest48 + 0x9E3779B97F4A7C15 * (j + 1)) & ((1 << 64) - 1)
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & ((1 << 64) - 1)
    return (x ^ (x >> 31)) & ((1 << 30) - 1)


@dataclass
class PreparedChat:
    ids: List[int]                       # scheduler-side ids (image positions carry pseudo ids >= vocab)
    real_ids: List[int]                  # the same prompt with the pad id at image positions (sampler token counts)
    spans: List[Tuple[int, torch.Tensor]]   # (first position, rows [tokens, hidden]) per image
    image_tokens: int = 0


class VisionFrontend:
    def __init__(self, tower, spec: VisionSpec, vocab: int):
        self.tower, self.spec, self.vocab = tower, spec, vocab
        assert spec.preprocess.grid == tower.cfg.grid, "the processor grid must be patch x merge of the tower"

    def has_images(self, messages: list) -> bool:
        return any(p.get("type") == "image_url" for m in messages for p in m.get("parts") or ())

    def encode_image(self, image_url, param: str) -> Tuple[torch.Tensor, int]:
        """-> (rows [tokens, hidden] on the tower's device, 48-bit content hash of the canvas)."""
        canvas = prepare_image(image_url, self.spec.preprocess, param)
        h = int.from_bytes(hashlib.blake2b(canvas.tobytes() + repr(canvas.shape).encode(), digest_size=6).digest(), "big")
        dev = self.tower.patch_embed.payload.device
        t = torch.from_numpy(canvas).to(dev)
        rows = self.tower.forward(t) if dev.type == "cuda" else self.tower.forward_reference(t)
        return rows, h

    def prepare_chat(self, messages: list, render: Callable[[list], str], encode: Callable[[str], List[int]]) -> PreparedChat:
        """messages: the validated message list (image messages carry their ordered `parts`).  render(messages) ->
        prompt text; encode(text) -> token ids."""
        images = []                                  # (param, image_url value)
        flat = []
        for mi, m in enumerate(messages):
            parts = m.get("parts")
            if not parts:
                flat.append({k: v for k, v in m.items() if k != "parts"})
                continue
            text = ""
            for pi, part in enumerate(parts):
                typ = part.get("type")
                if typ == "text":
                    text += part["text"].replace(SENTINEL, "")
                elif typ == "image_url":
                    if m.get("role") != "user":
                        raise ImageInputError("images are accepted in user messages only", f"messages[{mi}].content[{pi}]")
                    if len(images) >= MAX_IMAGES_PER_REQUEST:
                        raise ImageInputError(f"at most {MAX_IMAGES_PER_REQUEST} images per request",
                                              f"messages[{mi}].content[{pi}]")
                    text += f"{SENTINEL}{len(images)}{SENTINEL}"
                    images.append((f"messages[{mi}].content[{pi}].image_url", part.get("image_url")))
                else:
                    raise ImageInputError(f"content parts of type '{typ}' are not supported by this model",
                                          f"messages[{mi}].content[{pi}]")
            mm = {k: v for k, v in m.items() if k != "parts"}
            mm["content"] = text
            flat.append(mm)
        pieces = render(flat).split(SENTINEL)
        # pieces alternate text, image index, text, ... (user text cannot contain the sentinel any more)
        if len(pieces) != 2 * len(images) + 1:
            raise ImageInputError("the chat template dropped or duplicated an image placeholder", "messages")
        ids: List[int] = []
        real: List[int] = []
        spans = []
        total = 0
        sp = self.spec
        for i, piece in enumerate(pieces):
            if i % 2 == 0:
                t = encode(piece) if piece else []
                ids += t
                real += t
                continue
            param, value = images[int(piece)]
            rows, h = self.encode_image(value, param)
            n = rows.shape[0]
            ids.append(sp.start_id)
            real.append(sp.start_id)
            spans.append((len(ids), rows))
            # position j carries 30 bits of a position-dependent remix of the FULL 48-bit content digest, so the block
            # hashes of the span depend on all of its bits (a single 30-bit id per image would truncate it)
            ids += [self.vocab + _remix(h, j) for j in range(n)]
            real += [sp.pad_id] * n
            ids.append(sp.end_id)
            real.append(sp.end_id)
            total += n
        return PreparedChat(ids, real, spans, total)
