"""Host-side text preparation the engine's render/stream loops need: cleaning a
prompt and cutting it into the per-chunk turns the model was trained on.

Behaviour follows ``simple_clean`` and ``chunk_text`` of the reference
(src/vui/inference.py:88-132, 408-472 in fluxions-ai/vui); this is string
handling on the host, not part of the accelerated path.
"""

from __future__ import annotations

import re

# non-speech tags the tokenizer knows (src/vui/tokenizer.py:60-82, bracketed entries)
NON_SPEECH_TAGS = frozenset(
    "[pause] [hesitate] [breath] [env] [tut] [mouthnoise] [sigh] [scoff] [gasp] [sniff] [music] "
    "[sing] [laugh] [cough] [clearsthroat] [noise] [overlap] [SC] [shortpause] [longpause]".split()
)

_SENTENCE_END = re.compile(r'[.!?]+(?:["\'\)\]]+)?(?=\s|\[|$)')
_TAG_AT_END = re.compile(r"\[.*?\]\s*$")


def _pad_tags(text: str) -> str:
    """Put whitespace around [tags] (keeping an adjacent newline a newline)."""

    def before(m):
        return ("\n" if m.start() > 0 and text[m.start() - 1] == "\n" else " ") + m.group(1)

    out = re.sub(r"(?<![<\[\s])(\[)", before, text)
    src = out

    def after(m):
        return m.group(1) + ("\n" if m.end() < len(src) and src[m.end()] == "\n" else " ")

    return re.sub(r"(?<!\d\])(\])(?![>\]\s])", after, src).strip()


def _drop_unknown_tags(text: str) -> str:
    for inner in re.findall(r"\[([^\]]+)\]", text):
        tag = f"[{inner}]"
        if tag not in NON_SPEECH_TAGS:
            text = text.replace(tag, "")
    return text


def simple_clean(text: str) -> str:
    text = re.sub(r"(\d+)am", r"\1 AM", text)
    text = re.sub(r"(\d+)pm", r"\1 PM", text)
    text = _drop_unknown_tags(_pad_tags(text))
    for a, b in (("’", "'"), ("‘", "'"), ("”", '"'), ("“", '"')):
        text = text.replace(a, b)
    # a quote that is not inside a word is a wrapping quote: drop it with the double quotes
    text = re.sub(r"(?<![A-Za-z])'|'(?![A-Za-z])", '"', text).replace('"', "")
    text = text.replace("%", " percent").replace("*", "")
    text = re.sub(r"\([^)]*\)", "", text).replace("(", "").replace(")", "")
    text = text.replace(";", "").replace("–", " ").replace("—", "")
    text = re.sub(r"(?<!\w)-|-(?!\w)", "", text)  # hyphens that do not join two word characters
    text = text.replace(":", "").replace("…", "...").replace("s...", "s")
    text = re.sub(r"\bvs\.?\b", "versus", text, flags=re.IGNORECASE)
    text = re.sub(r"\n+", "\n", text)
    text = re.sub(r"[ \t]+", " ", text)
    text = re.sub(r" *\n *", "\n", text).strip()
    if not text.endswith((".", "?")):
        text += "."
    return text


def _split_sentences(text: str, max_words: int) -> list[str]:
    pieces, rest = [], text
    while rest:
        m = _SENTENCE_END.search(rest)
        if m:
            head, rest = rest[: m.end()].strip(), rest[m.end():].lstrip()
        else:
            words = rest.split()
            if len(words) > max_words:
                head, rest = " ".join(words[:max_words]).rstrip(",;:"), " ".join(words[max_words:])
            else:
                head, rest = rest.strip(), ""
        if head:
            pieces.append(head)
    return pieces


def chunk_text(text: str, min_words: int = 5, sentence_only: bool = False,
               single_speaker: bool = False) -> list[dict]:
    """Cut ``text`` into chunks ``{"text": str, "sc": bool}``.  A newline or an
    explicit ``[SC]`` starts a new speaker (``sc`` true on that speaker's first
    chunk unless ``single_speaker``).  Inside one speaker's line, clauses are cut
    after ``.!?`` and before ``, `` and merged until each has ``min_words`` words;
    with ``sentence_only`` only sentence ends cut, with a hard cut every
    ``min_words`` words for a sentence that never ends."""
    lines = []
    for raw in text.strip().split("\n"):
        raw = raw.strip()
        if not raw:
            continue
        for i, part in enumerate(re.split(r"\[SC\]", raw)):
            if part.strip():
                lines.append((part.strip(), i > 0))
    chunks: list[dict] = []
    for li, (line, explicit) in enumerate(lines):
        line = simple_clean(line)
        new_speaker = (li > 0 or explicit) and not single_speaker
        if sentence_only:
            parts = _split_sentences(line, min_words)
        else:
            clauses = [c.strip() for c in re.split(r"(?<=[.!?])\s+|\s*,\s+", line) if c.strip()]
            merged: list[str] = []
            for c in clauses:
                if merged and len(merged[-1].split()) < min_words:
                    merged[-1] += " " + c
                else:
                    merged.append(c)
            if len(merged) > 1 and len(merged[-1].split()) < min_words:
                tail = merged.pop()
                merged[-1] += " " + tail
            parts = []
            for m in merged:
                m = m.rstrip(",").rstrip()
                if parts and _TAG_AT_END.search(parts[-1]):
                    parts[-1] += " " + m  # never end a chunk on a [tag]
                else:
                    parts.append(m)
        first = True
        for p in parts:
            if p:
                chunks.append({"text": p, "sc": new_speaker and first})
                first = False
    return chunks
