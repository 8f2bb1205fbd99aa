"""Tokenizer front end, offline HF-hub helpers and grammar-constrained decoding.

* ``load_tokenizer / encode / decode / apply_chat_template`` wrap the ``tokenizers`` library
  (ferrotorch-tokenize/src/lib.rs).
* ``HfTransformerConfig`` parses a ``config.json``; ``hf_cache_path`` resolves a model directory in
  the local HF cache (``HF_HOME``); downloads are not available offline, so ``hf_download_model``
  only returns an existing snapshot (ferrotorch-hub/src/{hf_config,download}.rs).
* ``JsonGrammar`` + ``token_mask`` / ``apply_token_mask``: a JSON prefix validator drives a per-step
  mask over the vocabulary so that generation can only produce valid JSON
  (ferrotorch-grammar/src/state.rs; the mask is applied on the logits' device like the
  reference's ``compute_mask_gpu`` / ``kernel_apply_token_mask``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import torch


# --------------------------------------------------------------------------- tokenizer
def load_tokenizer(path: str):
    from tokenizers import Tokenizer

    return Tokenizer.from_file(path)


def encode(tok, text: str, add_special_tokens: bool = True) -> list[int]:
    return tok.encode(text, add_special_tokens=add_special_tokens).ids


def decode(tok, ids, skip_special_tokens: bool = True) -> str:
    return tok.decode(list(ids), skip_special_tokens=skip_special_tokens)


def apply_chat_template(messages: list[dict], template: str = "llama3", add_generation_prompt: bool = True) -> str:
    """Render ``[{"role": ..., "content": ...}]`` with the Llama-3 or ChatML layout."""
    if template == "llama3":
        out = "<|begin_of_text|>"
        for m in messages:
            out += "<|start_header_id|>%s<|end_header_id|>\n\n%s<|eot_id|>" % (m["role"], m["content"])
        return out + ("<|start_header_id|>assistant<|end_header_id|>\n\n" if add_generation_prompt else "")
    if template == "chatml":
        out = "".join("<|im_start|>%s\n%s<|im_end|>\n" % (m["role"], m["content"]) for m in messages)
        return out + ("<|im_start|>assistant\n" if add_generation_prompt else "")
    raise ValueError("unknown chat template %r" % template)


# --------------------------------------------------------------------------- hub (offline)
@dataclass
class HfTransformerConfig:
    model_type: str = "llama"
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_file(cls, path: str) -> "HfTransformerConfig":
        with open(path) as f:
            raw = json.load(f)
        return cls(raw.get("model_type", "unknown"), raw)

    def to_llama(self):
        from ..models.llama import LlamaConfig

        return LlamaConfig.from_hf(self.raw)


def hf_cache_path(repo_id: str) -> str:
    home = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
    return os.path.join(home, "hub", "models--" + repo_id.replace("/", "--"))


def hf_download_model(repo_id: str) -> str:
    """Return the newest local snapshot of ``repo_id``; raises when it is not cached (no network)."""
    snaps = os.path.join(hf_cache_path(repo_id), "snapshots")
    if not os.path.isdir(snaps) or not os.listdir(snaps):
        raise FileNotFoundError("%s is not in the local HF cache and downloads are unavailable offline" % repo_id)
    return os.path.join(snaps, sorted(os.listdir(snaps))[-1])


# --------------------------------------------------------------------------- JSON grammar
class JsonGrammar:
    """Incremental validator: ``accepts_prefix(s)`` is True iff ``s`` can be extended to valid JSON
    (a value of the kinds in ``allow``), ``is_complete(s)`` iff it already is one."""

    WS = " \t\n\r"

    def __init__(self, allow=("object", "array", "string", "number", "true", "false", "null")):
        self.allow = set(allow)

    def is_complete(self, s: str) -> bool:
        try:
            json.loads(s)
            return True
        except ValueError:
            return False

    def accepts_prefix(self, s: str) -> bool:
        st = self._scan(s)
        return st is not None

    def _scan(self, s: str):
        """Returns a stack description if ``s`` is a valid prefix, else None."""
        stack: list[str] = []      # "{k" expect key, "{:" expect colon, "{v" expect value, "{," after value; "[v", "[,"
        i, n, done = 0, len(s), False
        expect_value = True

        def after_value():
            nonlocal done, expect_value
            expect_value = False
            if not stack:
                done = True
            elif stack[-1] in ("{v",):
                stack[-1] = "{,"
            elif stack[-1] == "[v":
                stack[-1] = "[,"

        while i < n:
            c = s[i]
            if c in self.WS:
                i += 1
                continue
            if done:
                return None
            top = stack[-1] if stack else None
            if expect_value and top != "{k":
                if c == "{":
                    stack.append("{k")
                    expect_value = False
                    i += 1
                elif c == "[":
                    stack.append("[v")
                    i += 1
                elif c == "]" and top == "[v" and s[:i].rstrip()[-1:] == "[":
                    stack.pop()
                    after_value()
                    i += 1
                elif c == '"':
                    j = self._string_end(s, i)
                    if j is None:
                        return stack if self._string_prefix_ok(s[i:]) else None
                    i = j
                    after_value()
                elif c in "-0123456789":
                    j = i + 1
                    while j < n and s[j] in "0123456789+-.eE":
                        j += 1
                    tok = s[i:j]
                    if j == n:
                        return stack if self._number_prefix_ok(tok) else None
                    try:
                        float(tok)
                    except ValueError:
                        return None
                    if tok in ("-",) or (len(tok) > 1 and tok[0] == "0" and tok[1].isdigit()):
                        return None
                    i = j
                    after_value()
                else:
                    for lit in ("true", "false", "null"):
                        if lit.startswith(s[i:i + len(lit)]) and s[i:i + len(lit)]:
                            if len(s) - i < len(lit):
                                return stack if lit.startswith(s[i:]) else None
                            if s[i:i + len(lit)] == lit:
                                i += len(lit)
                                after_value()
                                break
                    else:
                        return None
                continue
            if top == "{k":
                if c == "}" and s[:i].rstrip()[-1:] == "{":
                    stack.pop()
                    after_value()
                    i += 1
                elif c == '"':
                    j = self._string_end(s, i)
                    if j is None:
                        return stack if self._string_prefix_ok(s[i:]) else None
                    i = j
                    stack[-1] = "{:"
                else:
                    return None
            elif top == "{:":
                if c != ":":
                    return None
                stack[-1] = "{v"
                expect_value = True
                i += 1
            elif top == "{,":
                if c == ",":
                    stack[-1] = "{k"
                elif c == "}":
                    stack.pop()
                    after_value()
                else:
                    return None
                i += 1
            elif top == "[,":
                if c == ",":
                    stack[-1] = "[v"
                    expect_value = True
                elif c == "]":
                    stack.pop()
                    after_value()
                else:
                    return None
                i += 1
            else:
                return None
        return stack

    @staticmethod
    def _string_end(s: str, i: int):
        j = i + 1
        while j < len(s):
            if s[j] == "\\":
                j += 2
                continue
            if s[j] == '"':
                return j + 1
            if ord(s[j]) < 0x20:
                return None
            j += 1
        return None

    @staticmethod
    def _string_prefix_ok(s: str) -> bool:
        return all(ord(c) >= 0x20 for c in s)

    @staticmethod
    def _number_prefix_ok(tok: str) -> bool:
        if tok in ("-",):
            return True
        if len(tok) > 1 and tok.lstrip("-")[:1] == "0" and tok.lstrip("-")[1:2].isdigit():
            return False
        try:
            float(tok)
            return True
        except ValueError:
            try:
                float(tok + "0")
                return True
            except ValueError:
                return False


def token_mask(grammar: JsonGrammar, generated: str, vocab: list[str], eos_id: int | None = None,
               device=None) -> torch.Tensor:
    """Boolean mask ``[len(vocab)]`` of tokens that keep ``generated`` a valid JSON prefix; EOS is
    allowed once the text is a complete value."""
    mask = torch.zeros(len(vocab), dtype=torch.bool)
    for i, piece in enumerate(vocab):
        if i == eos_id:
            mask[i] = grammar.is_complete(generated)
        elif piece:
            mask[i] = grammar.accepts_prefix(generated + piece)
    return mask.to(device) if device is not None else mask


def apply_token_mask(logits: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Set disallowed logits to -inf on the logits' device."""
    return logits.masked_fill(~mask.to(logits.device), float("-inf"))
