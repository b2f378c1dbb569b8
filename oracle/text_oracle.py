"""CPU oracle for token-ids -> text/timestamps.  TEST INFRASTRUCTURE ONLY.

Restates, for small cases, the reference's
  ParakeetTdtDecoder::decode      src/decode.rs:39-104
  frame_to_seconds                src/decode.rs:106-108
  is_special_token                src/decode.rs:110-112
  needs_digit_spacing             src/decode.rs:114-134
  Vocabulary::from_file           src/vocab.rs:15-52
  join_token_text / build_chunk / build_result   src/long_form.rs:602-647
Pinned by the reference's known-answer tests decode.rs:151-179.
Rust's `char::is_alphabetic` is the Unicode derived property Alphabetic; the `regex` package's `\\p{Alphabetic}`
(Unicode 17.0 tables) stands in for it here.
"""
from __future__ import annotations

import regex

_ALPHABETIC = regex.compile(r"\p{Alphabetic}")

SECONDS_PER_FRAME = 1280 / 16000


def parse_vocab(text: str):
    """vocab.rs:15-52: lines of '<token> <id>'; blank = id of <blk>/<blank>, else the last id."""
    id_to_token: list[str] = []
    blank = None
    for line in text.split("\n"):
        if line.endswith("\r"):
            line = line[:-1]
        parts = line.split(" ", 1)
        if len(parts) < 2:
            continue
        token, idx = parts
        if not idx.isdigit() and not (idx.startswith("+") and idx[1:].isdigit()):
            raise ValueError(f"invalid token id `{idx}`")
        i = int(idx)
        if i >= len(id_to_token):
            id_to_token.extend([""] * (i + 1 - len(id_to_token)))
        id_to_token[i] = token
        if token in ("<blk>", "<blank>"):
            blank = i
    if not id_to_token:
        raise ValueError("vocabulary was empty")
    return id_to_token, (blank if blank is not None else len(id_to_token) - 1)


def frame_to_seconds(frame: int) -> float:
    return (frame * 160 * 8) / 16000


def is_special_token(tok: str) -> bool:
    return tok.startswith("<") and tok.endswith(">") and tok != "<unk>"


def needs_digit_spacing(existing: str, display: str) -> bool:
    if existing == "" or display.startswith(" "):
        return False
    if not all(ch in "0123456789" for ch in display):
        return False
    trailing = 0
    for ch in reversed(existing):
        if _ALPHABETIC.match(ch):
            trailing += 1
        else:
            break
    is_article_a = trailing == 1 and existing[-1] == "a"
    return trailing > 1 or is_article_a


def decode(vocab: list[str], token_ids, frames, confidences, duration_seconds: float):
    """Returns dict(text, chunks=[(start,end,text)], tokens=[(id,text,start,end,conf)], duration_seconds)."""
    if len(token_ids) == 0:
        return dict(text="", chunks=[], tokens=[], duration_seconds=duration_seconds)
    text = ""
    tokens = []
    for index, tid in enumerate(token_ids):
        tid = int(tid)
        if tid >= len(vocab):
            continue
        tok = vocab[tid]
        if is_special_token(tok):
            continue
        start = frame_to_seconds(int(frames[index]))
        if index + 1 < len(frames):
            end = frame_to_seconds(int(frames[index + 1]))
        else:
            end = min(start + SECONDS_PER_FRAME, duration_seconds)
        display = tok.replace("▁", " ")
        if needs_digit_spacing(text, display):
            display = " " + display
        text += display
        conf = float(confidences[index]) if index < len(confidences) else 0.0
        tokens.append((tid, display, start, end, conf))
    text = text.strip()
    chunks = []
    if text and tokens:
        chunks = [(tokens[0][2], tokens[-1][3], text)]
    return dict(text=text, chunks=chunks, tokens=tokens, duration_seconds=duration_seconds)


def long_form_result(tokens, audio_len: int):
    """long_form.rs:344-374,602-647 for one Overlap region: chunk text is re-joined
    from the token texts and trimmed; result text joins chunk texts with ' '."""
    chunks = []
    if tokens:
        joined = "".join(t[1] for t in tokens).strip()
        chunks = [(tokens[0][2], tokens[-1][3], joined)]
    else:
        tokens = []
    text = " ".join(c[2] for c in chunks)
    return dict(text=text, chunks=chunks, tokens=list(tokens), duration_seconds=audio_len / 16000)
