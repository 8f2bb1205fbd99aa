"""Tokenizer front end, offline HF-hub helpers and grammar-constrained decoding.

* ``load_tokenizer / encode / decode / apply_chat_template`` wrap the ``tokenizers`` library
  (ferrotorch-tokenize/src/lib.rs).
* ``HfTransformerConfig`` parses a ``config.json``; ``hf_cache_path`` resolves a model directory in
  the local HF cache (``HF_HOME``); downloads are not available offline, so ``hf_download_model``
  only returns an existing snapshot (ferrotorch-hub/src/{hf_config,download}.rs).
* ``JsonGrammar`` + ``token_mask`` / ``apply_token_mask``: a JSON prefix validator drives a per-step
  mask over the vocabulary so that generation can only produce valid JSON
  (ferrotorch-grammar/src/state.rs; the mask is applied on the logits' device like the
  reference's ``compute_mask_gpu`` / ``kernel_apply_token_mask``).  Decoding under a JSON *schema*
  (``JsonSchemaProcessor``, ``TokenMask``, ``TokenTransitionCache``) lives in ``utils.grammar``.
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


def encode_batch(tok, texts: list[str], add_special_tokens: bool = True) -> list[list[int]]:
    return [e.ids for e in tok.encode_batch(list(texts), add_special_tokens=add_special_tokens)]


def vocab_size(tok, with_added_tokens: bool = True) -> int:
    return tok.get_vocab_size(with_added_tokens=with_added_tokens)


def token_to_id(tok, token: str) -> int | None:
    return tok.token_to_id(token)


def id_to_token(tok, idx: int) -> str | None:
    return tok.id_to_token(idx)


@dataclass
class ChatMessage:
    """One turn; ``extra`` carries whatever else a template reads (``tool_calls``, ``name`` ...)
    and is flattened next to ``role`` / ``content`` (ferrotorch-tokenize/src/lib.rs:203-225)."""
    role: str
    content: str
    extra: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {**self.extra, "role": self.role, "content": self.content}


_BUILTIN_TEMPLATES = {
    "llama3": ("{{ bos_token if bos_token else '<|begin_of_text|>' }}"
               "{% for m in messages %}<|start_header_id|>{{ m['role'] }}<|end_header_id|>\n\n{{ m['content'] }}<|eot_id|>{% endfor %}"
               "{% if add_generation_prompt %}<|start_header_id|>assistant<|end_header_id|>\n\n{% endif %}"),
    "chatml": ("{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
               "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"),
}


def apply_chat_template(messages, template: str = "llama3", add_generation_prompt: bool = True,
                        bos_token: str | None = None, eos_token: str | None = None) -> str:
    """Render a conversation with a Jinja chat template, the kind ``tokenizer_config.json`` carries
    (ferrotorch-tokenize/src/lib.rs:247-330: variables ``messages``, ``add_generation_prompt``,
    ``bos_token``, ``eos_token``; helpers ``raise_exception(msg)`` and ``strftime_now(fmt)``).
    ``template`` is the template text, or ``"llama3"`` / ``"chatml"`` for the two built-in layouts.
    Messages are dicts or :class:`ChatMessage`.  Templates run in Jinja's sandbox."""
    import datetime

    import jinja2
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(msg):
        raise jinja2.exceptions.TemplateError(msg)

    def strftime_now(fmt):
        return datetime.datetime.now().strftime(fmt)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
    env.globals.update(raise_exception=raise_exception, strftime_now=strftime_now)
    text = _BUILTIN_TEMPLATES.get(template, template)
    try:
        tmpl = env.from_string(text)
    except jinja2.exceptions.TemplateSyntaxError as e:
        raise ValueError("invalid chat template: %s" % e)
    msgs = [m.to_dict() if isinstance(m, ChatMessage) else dict(m) for m in messages]
    try:
        return tmpl.render(messages=msgs, add_generation_prompt=add_generation_prompt, bos_token=bos_token or "",
                           eos_token=eos_token or "")
    except jinja2.exceptions.TemplateError as e:
        raise ValueError("chat template render failed: %s" % e)


def apply_chat_template_to_ids(tok, template: str, messages, add_generation_prompt: bool = True,
                               bos_token: str | None = None, eos_token: str | None = None,
                               add_special_tokens: bool = False) -> tuple[str, list[int]]:
    """Render, then tokenise: ``(prompt, ids)``."""
    prompt = apply_chat_template(messages, template, add_generation_prompt, bos_token, eos_token)
    return prompt, encode(tok, prompt, add_special_tokens)


def load_chat_template(tokenizer_config_path: str) -> str | None:
    """The ``chat_template`` of a ``tokenizer_config.json``: a string, or the first entry of a list
    of ``{"name", "template"}`` objects; ``None`` when the file has none."""
    with open(tokenizer_config_path, "rb") as f:
        data = f.read()
    try:
        value = json.loads(data)
    except ValueError as e:
        raise ValueError("failed to parse tokenizer_config %s: %s" % (tokenizer_config_path, e))
    t = value.get("chat_template") if isinstance(value, dict) else None
    if t is None or isinstance(t, str):
        return t
    if isinstance(t, list):
        for entry in t:
            if isinstance(entry, dict) and isinstance(entry.get("template"), str):
                return entry["template"]
        return None
    raise ValueError("tokenizer_config %s has chat_template of unexpected type" % tokenizer_config_path)


# --------------------------------------------------------------------------- hub (offline)
@dataclass
class HfTransformerConfig:
    """The fields of a Hugging Face ``config.json`` that a decoder-only transformer needs
    (ferrotorch-hub/src/hf_config.rs:60-120), with the same defaults: ``rms_norm_eps`` 1e-6,
    ``rope_theta`` 10000, ``hidden_act`` "silu", untied embeddings.  ``raw`` keeps everything."""
    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads_: int | None = None
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 0
    vocab_size: int = 0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    hidden_act_param: float | None = None
    torch_dtype: str | None = None
    architectures: list = field(default_factory=list)
    rope_scaling: dict | None = None
    model_type: str | None = None
    raw: dict = field(default_factory=dict)

    _REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                 "max_position_embeddings", "vocab_size")

    @classmethod
    def from_dict(cls, raw: dict) -> "HfTransformerConfig":
        missing = [k for k in cls._REQUIRED if k not in raw]
        if missing:
            raise ValueError("failed to parse HF config JSON: missing field(s) %s" % ", ".join(missing))
        kw = {k: raw[k] for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                  "rms_norm_eps", "rope_theta", "max_position_embeddings", "vocab_size",
                                  "tie_word_embeddings", "hidden_act", "hidden_act_param", "torch_dtype",
                                  "architectures", "rope_scaling", "model_type") if raw.get(k) is not None}
        rp = raw.get("rope_parameters")
        if isinstance(rp, dict):                      # newer files: rotary settings in one object
            if "rope_theta" not in kw and "rope_theta" in rp:
                kw["rope_theta"] = rp["rope_theta"]
            if "rope_scaling" not in kw and rp.get("rope_type", "default") != "default":
                kw["rope_scaling"] = rp
        return cls(num_key_value_heads_=raw.get("num_key_value_heads"), raw=dict(raw), **kw)

    @classmethod
    def from_json_str(cls, s: str) -> "HfTransformerConfig":
        try:
            raw = json.loads(s)
        except ValueError as e:
            raise ValueError("failed to parse HF config JSON: %s" % e)
        if not isinstance(raw, dict):
            raise ValueError("failed to parse HF config JSON: not an object")
        return cls.from_dict(raw)

    @classmethod
    def from_file(cls, path: str) -> "HfTransformerConfig":
        with open(path, encoding="utf-8") as f:
            return cls.from_json_str(f.read())

    def num_key_value_heads(self) -> int:
        return self.num_key_value_heads_ if self.num_key_value_heads_ is not None else self.num_attention_heads

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def is_gqa(self) -> bool:
        return self.num_key_value_heads() < self.num_attention_heads

    def validate(self) -> None:
        if min(self.hidden_size, self.num_attention_heads, self.num_hidden_layers, self.intermediate_size,
               self.vocab_size) <= 0:
            raise ValueError("HfTransformerConfig: hidden_size / num_attention_heads / num_hidden_layers / "
                             "intermediate_size / vocab_size must all be positive")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("HfTransformerConfig: hidden_size (%d) must be divisible by num_attention_heads (%d)"
                             % (self.hidden_size, self.num_attention_heads))
        kv = self.num_key_value_heads()
        if kv <= 0 or self.num_attention_heads % kv:
            raise ValueError("HfTransformerConfig: num_attention_heads (%d) must be divisible by a positive "
                             "num_key_value_heads (%d)" % (self.num_attention_heads, kv))
        if self.hidden_act not in ("silu", "swish", "gelu", "gelu_new", "relu", "fatrelu"):
            raise ValueError("HfTransformerConfig: unsupported hidden_act %r (supported: silu, swish, gelu, "
                             "gelu_new, relu, fatrelu)" % (self.hidden_act,))

    def to_llama(self):
        from ..models.llama import LlamaConfig

        self.validate()
        raw = dict(self.raw)
        raw.setdefault("rms_norm_eps", self.rms_norm_eps)
        raw.setdefault("rope_theta", self.rope_theta)
        return LlamaConfig.from_hf(raw)


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


def __getattr__(name):
    """``Tokenizer`` is the Hugging Face ``tokenizers`` class itself, imported on first use."""
    if name == "Tokenizer":
        from tokenizers import Tokenizer

        return Tokenizer
    raise AttributeError(name)
