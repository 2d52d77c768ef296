"""Renderers turn a raw record into SEGMENTS: ``[(text, trained), ...]``. The packer tokenises every
segment separately, so whether a span contributes to the loss is decided here, per role, not by string
surgery on token ids. Reference: src/kohakuwullm/data/renderers (plain.py, chatml.py, tipo.py)."""

from __future__ import annotations

import random
from typing import Callable, Sequence

from kohakuwullm_b200.registry import RENDERER

Segment = tuple[str, bool]

CHAT_SPECIALS = ("<|im_start|>", "<|im_end|>", "<|system|>", "<|user|>", "<|assistant|>", "<|tool|>",
                 "<|think|>", "<|/think|>")
CHATML_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"
)


@RENDERER.register("plain")
class PlainRenderer:
    """The whole text is one trained segment."""

    def __init__(self, field: str = "text", **_unused):
        self.field = field

    def __call__(self, record, rng: random.Random | None = None) -> list[Segment]:
        text = record if isinstance(record, str) else record.get(self.field, "")
        return [(text, True)]


@RENDERER.register("chatml")
class ChatMLRenderer:
    """``<|im_start|>role\\ncontent<|im_end|>\\n`` per turn; only ``trained_roles`` contribute to the loss
    (the closing ``<|im_end|>`` of a trained turn is trained so the model learns to stop)."""

    def __init__(self, trained_roles: Sequence[str] = ("assistant",), field: str = "messages", **_unused):
        self.trained_roles, self.field = set(trained_roles), field

    def __call__(self, record, rng=None) -> list[Segment]:
        segs: list[Segment] = []
        for turn in record[self.field] if isinstance(record, dict) else record:
            role, content = turn["role"], turn["content"]
            trained = role in self.trained_roles
            segs.append((f"<|im_start|>{role}\n", False))
            segs.append((f"{content}<|im_end|>\n", trained))
        return segs


RENDERER.register("chat", ChatMLRenderer)


@RENDERER.register("qa_chatml")
class QAChatMLRenderer(ChatMLRenderer):
    """Question/answer records rendered as a two-turn chat."""

    def __init__(self, question: str = "question", answer: str = "answer", system: str | None = None, **kw):
        super().__init__(**kw)
        self.q, self.a, self.system = question, answer, system

    def __call__(self, record, rng=None) -> list[Segment]:
        msgs = []
        if self.system:
            msgs.append({"role": "system", "content": self.system})
        msgs += [{"role": "user", "content": record[self.q]}, {"role": "assistant", "content": record[self.a]}]
        return super().__call__(msgs)


@RENDERER.register("tipo")
class TIPORenderer:
    """Text-to-image prompt records (tag lists + optional natural-language captions) rendered as one of
    several tasks — tags->caption, caption->tags, short->long tags, ... — chosen by the injected rng, with
    a target-length bucket token. The metadata/prefix is context; the completion is trained."""

    TASKS = ("tag_to_long", "long_to_tag", "short_to_tag", "tag_to_short", "short_to_long", "short_to_tag_to_long",
             "tag_to_short_to_long", "gen_meta")
    LENGTHS = ("very_short", "short", "long", "very_long")

    def __init__(self, tasks: Sequence[str] | None = None, **_unused):
        self.tasks = tuple(tasks or self.TASKS)

    @staticmethod
    def length_bucket(n_tags: int) -> str:
        return TIPORenderer.LENGTHS[0 if n_tags < 10 else 1 if n_tags < 25 else 2 if n_tags < 45 else 3]

    def build_prompt(self, record, task: str, rng: random.Random) -> tuple[str, str]:
        tags = list(record.get("tags", []))
        rng.shuffle(tags)
        caption = record.get("caption", "")
        short = record.get("short_caption", caption.split(".")[0] if caption else "")
        meta = ", ".join(f"{k}: {record[k]}" for k in ("rating", "artist", "characters", "aspect_ratio") if record.get(k))
        cut = max(1, len(tags) // 3)
        head = f"{meta}\ntarget: <|{self.length_bucket(len(tags))}|>\n" if meta else f"target: <|{self.length_bucket(len(tags))}|>\n"
        table = {
            "tag_to_long": (f"{head}tags: {', '.join(tags)}\nlong: ", caption),
            "long_to_tag": (f"{head}long: {caption}\ntags: ", ", ".join(tags)),
            "short_to_tag": (f"{head}short: {short}\ntags: ", ", ".join(tags)),
            "tag_to_short": (f"{head}tags: {', '.join(tags)}\nshort: ", short),
            "short_to_long": (f"{head}short: {short}\nlong: ", caption),
            "short_to_tag_to_long": (f"{head}short: {short}\ntags: ", f"{', '.join(tags)}\nlong: {caption}"),
            "tag_to_short_to_long": (f"{head}tags: {', '.join(tags[:cut])}\nshort: ", f"{short}\nlong: {caption}"),
            "gen_meta": (head + "tags: " + ", ".join(tags[:cut]), ", " + ", ".join(tags[cut:]) if len(tags) > cut else ""),
        }
        return table[task]

    def __call__(self, record, rng: random.Random | None = None) -> list[Segment]:
        rng = rng or random.Random(0)
        task = rng.choice(self.tasks)
        prompt, completion = self.build_prompt(record, task, rng)
        return [(prompt, False), (completion, True)]


@RENDERER.register("per_source")
class PerSourceRenderer:
    """Dispatch on ``record['source']`` to one of several renderers."""

    def __init__(self, renderers: dict[str, Callable], default: str | None = None, **_unused):
        from kohakuwullm_b200.registry import build

        self.renderers = {k: build(v, RENDERER) for k, v in renderers.items()}
        self.default = default

    def __call__(self, record, rng=None) -> list[Segment]:
        key = record.get("source", self.default)
        if key not in self.renderers:
            key = self.default
        return self.renderers[key](record, rng)
