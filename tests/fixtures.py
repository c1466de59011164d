"""Shared test fixtures: a small byte-level BPE tokenizer.json in the Hugging Face layout."""
import json


def bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b); cs.append(256 + n); n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


QWEN2_SPLIT = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>"]
PLAIN_ADDED = ["<think>", "</think>", "<tool_call>", "</tool_call>"]


def tiny_tokenizer_json() -> str:
    b2u = bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    merges = []
    G = b2u[ord(" ")]

    def add(a, b):
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)

    for a, b in [("t", "h"), ("th", "e"), (G, "t"), (G + "t", "he"), ("i", "n"), ("e", "r"), ("a", "n"), (G, "a"), ("o", "n"),
                 ("r", "e"), ("h", "e"), (G, "w"), ("l", "l"), ("he", "ll"), ("hell", "o"), (G + "w", "o"), ("in", "g"),
                 ("an", "d"), (G, G), (G + G, G + G), ("Ċ", "Ċ"), ("1", "2")]:
        add(a, b)
    added = []
    nid = len(vocab)
    for s in SPECIALS:
        added.append({"id": nid, "content": s, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True}); nid += 1
    for s in PLAIN_ADDED:
        added.append({"id": nid, "content": s, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": False}); nid += 1
    tj = {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": added, "normalizer": None,
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": QWEN2_SPLIT}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False}]},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": "", "end_of_word_suffix": "",
                  "fuse_unk": False, "byte_fallback": False, "ignore_merges": False, "vocab": vocab, "merges": merges},
    }
    return json.dumps(tj)
