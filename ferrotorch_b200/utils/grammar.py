"""JSON-Schema-constrained decoding: a schema compiler, a character-level matcher, and a token-mask
processor that plugs into ``generate``.

The reference's ``ferrotorch-grammar`` crate does the same job (schema.rs: the supported subset;
state.rs: a character-level state machine with ``valid_next_chars`` / ``step_char`` /
``is_complete``; json_schema.rs: ``JsonSchemaProcessor`` that admits a token iff all of its
characters are accepted in sequence, ``TokenMask``, ``TokenTransitionCache``).  The design here
differs in two ways:

* the matcher is **non-deterministic**: its state is a set of frame stacks, so ``oneOf`` /
  ``anyOf`` / ``enum`` branches whose first characters overlap stay alive until the text tells them
  apart (the reference commits to the first branch whose start accepts the character,
  schema.rs:33-41);
* the token mask is computed by walking a **trie of the vocabulary** once per matcher state, so
  tokens that share a prefix share the work, and masks are cached per state; the walk itself runs in
  C++ (``csrc/host/grammar_mask.cpp``) and calls back into the matcher only for (state, character)
  pairs it has not seen, with a pure-Python walk as the fallback.

Supported schema keywords: ``type`` (object, array, string, number, integer, boolean, null, or a
list of them), ``properties`` + ``required`` (only listed properties may appear, in any order),
``items`` / ``minItems`` / ``maxItems``, ``enum`` / ``const`` (any JSON scalars), ``minLength`` /
``maxLength``, ``minimum`` / ``maximum`` / ``multipleOf``, ``oneOf`` / ``anyOf``, and ``$ref`` into
``definitions`` / ``$defs`` (recursive references are rejected: the frame stack must stay
bounded).  ``allOf``, ``not`` and ``pattern`` raise :class:`SchemaError`; annotations are ignored.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

import torch


class SchemaError(ValueError):
    """The schema uses something outside the supported subset or is malformed."""


class GrammarError(ValueError):
    """A character or token that the grammar does not admit was fed to the matcher."""


# --------------------------------------------------------------------------- schema
@dataclass
class Node:
    kind: str                                   # object array string number integer literals union
    props: dict = field(default_factory=dict)   # object: name -> node id
    required: frozenset = frozenset()
    item: int = -1                              # array: node id of the element schema
    min_items: int = 0
    max_items: int | None = None
    min_len: int = 0                            # string
    max_len: int | None = None
    minimum: float | None = None                # number / integer
    maximum: float | None = None
    multiple_of: float | None = None
    literals: tuple = ()                        # literals: JSON texts (enum / const / true / false / null)
    branches: tuple = ()                        # union: node ids


_IGNORED = {"title", "description", "default", "examples", "format", "$schema", "$id", "$comment",
            "additionalProperties", "definitions", "$defs", "deprecated", "readOnly", "writeOnly"}
_UNSUPPORTED = ("allOf", "not", "pattern", "patternProperties", "if", "then", "else", "dependentSchemas")
MAX_DEPTH = 64


class Schema:
    """A compiled schema: ``nodes[root]`` describes the top-level value."""

    def __init__(self):
        self.nodes: list[Node] = []
        self.root = -1

    def _add(self, node: Node) -> int:
        self.nodes.append(node)
        return len(self.nodes) - 1

    @classmethod
    def from_json_schema(cls, value) -> "Schema":
        if isinstance(value, str):
            try:
                value = json.loads(value)
            except ValueError as e:
                raise SchemaError("schema is not valid JSON: %s" % e)
        s = cls()
        s.root = s._compile(value, value, 0, ())
        return s

    # -- helpers
    def _resolve(self, ref: str, root):
        if not isinstance(ref, str) or not ref.startswith("#/"):
            raise SchemaError("only references inside the document are supported, got %r" % (ref,))
        cur = root
        for part in ref[2:].split("/"):
            part = part.replace("~1", "/").replace("~0", "~")
            if not isinstance(cur, dict) or part not in cur:
                raise SchemaError("unresolvable reference %r" % ref)
            cur = cur[part]
        return cur

    def _literals(self, values) -> int:
        if not isinstance(values, list) or not values:
            raise SchemaError("enum must be a non-empty array")
        texts = []
        for v in values:
            if isinstance(v, (dict, list)):
                raise SchemaError("enum members must be scalars")
            t = json.dumps(v, ensure_ascii=False)
            if t not in texts:
                texts.append(t)
        return self._add(Node("literals", literals=tuple(texts)))

    def _compile(self, v, root, depth: int, active: tuple) -> int:
        if depth > MAX_DEPTH:
            raise SchemaError("schema nests deeper than %d levels" % MAX_DEPTH)
        if not isinstance(v, dict):
            raise SchemaError("a schema must be an object, got %s" % type(v).__name__)
        for k in _UNSUPPORTED:
            if k in v:
                raise SchemaError("keyword %r is not supported" % k)
        if "$ref" in v:
            ref = v["$ref"]
            if ref in active:
                raise SchemaError("recursive reference %r" % ref)
            return self._compile(self._resolve(ref, root), root, depth + 1, active + (ref,))
        if "const" in v:
            return self._literals([v["const"]])
        if "enum" in v:
            return self._literals(v["enum"])
        for key in ("oneOf", "anyOf"):
            if key in v:
                alts = v[key]
                if not isinstance(alts, list) or not alts:
                    raise SchemaError("%s must be a non-empty array" % key)
                return self._add(Node("union", branches=tuple(self._compile(a, root, depth + 1, active) for a in alts)))
        t = v.get("type")
        if t is None and "properties" in v:
            t = "object"
        if t is None and "items" in v:
            t = "array"
        if t is None:
            raise SchemaError("schema without a type: %s" % json.dumps(v)[:80])
        if isinstance(t, list):
            if not t:
                raise SchemaError("empty type list")
            ids = [self._compile(dict(v, type=one), root, depth + 1, active) for one in t]
            return ids[0] if len(ids) == 1 else self._add(Node("union", branches=tuple(ids)))
        return self._typed(t, v, root, depth, active)

    def _typed(self, t: str, v: dict, root, depth: int, active: tuple) -> int:
        def bound(key, kinds=(int, float)):
            x = v.get(key)
            if x is not None and (isinstance(x, bool) or not isinstance(x, kinds)):
                raise SchemaError("%s must be a number, got %r" % (key, x))
            return x

        def count(key):
            x = v.get(key)
            if x is not None and (isinstance(x, bool) or not isinstance(x, int) or x < 0):
                raise SchemaError("%s must be a non-negative integer, got %r" % (key, x))
            return x

        if t == "object":
            props = v.get("properties", {})
            if not isinstance(props, dict):
                raise SchemaError("properties must be an object")
            req = v.get("required", [])
            if not isinstance(req, list) or any(not isinstance(r, str) for r in req):
                raise SchemaError("required must be an array of strings")
            missing = [r for r in req if r not in props]
            if missing:
                raise SchemaError("required properties %s are not declared in properties" % missing)
            ids = {name: self._compile(sub, root, depth + 1, active) for name, sub in props.items()}
            return self._add(Node("object", props=ids, required=frozenset(req)))
        if t == "array":
            if "items" not in v:
                raise SchemaError("an array schema needs items")
            lo, hi = count("minItems") or 0, count("maxItems")
            if hi is not None and hi < lo:
                raise SchemaError("maxItems < minItems")
            return self._add(Node("array", item=self._compile(v["items"], root, depth + 1, active), min_items=lo,
                                  max_items=hi))
        if t == "string":
            lo, hi = count("minLength") or 0, count("maxLength")
            if hi is not None and hi < lo:
                raise SchemaError("maxLength < minLength")
            return self._add(Node("string", min_len=lo, max_len=hi))
        if t in ("number", "integer"):
            lo, hi, mul = bound("minimum"), bound("maximum"), bound("multipleOf")
            if mul is not None and mul <= 0:
                raise SchemaError("multipleOf must be positive")
            if lo is not None and hi is not None and hi < lo:
                raise SchemaError("maximum < minimum")
            return self._add(Node(t, minimum=lo, maximum=hi, multiple_of=mul))
        if t == "boolean":
            return self._add(Node("literals", literals=("true", "false")))
        if t == "null":
            return self._add(Node("literals", literals=("null",)))
        raise SchemaError("unsupported type %r" % (t,))


# --------------------------------------------------------------------------- matcher
# A state is a tuple of frames, innermost last; the empty tuple means "value complete".  Frames:
#   ("val", node)                         a value of schema `node` starts here
#   ("lit", suffixes)                     inside a literal: the candidates' remaining texts
#   ("str", lo, hi, n, esc)               inside a string body: n characters so far (saturates at lo
#                                         when there is no upper bound), esc = 0 plain, 1 after a
#                                         backslash, 2..5 = hex digits still owed by a \u escape
#   ("num", node, phase, text)            inside a number; text is kept only for constrained schemas
#   ("obj", node, seen, phase)            phase: "open" after {, "comma" after a comma, "after" after a value
#   ("key", node, seen, suffixes)         inside a property name: ((name, remaining text), ...)
#   ("colon", node, seen, name)           the name's closing quote is out, a colon is due
#   ("arr", node, n, phase)               phase: "open" after [, "comma", "after"; n elements begun
_WS = " \t\n\r"
_DIGITS = "0123456789"
_HEX = "0123456789abcdefABCDEF"
_NUM_DONE = ("0", "i", "f", "ed")


class _Machine:
    def __init__(self, schema: Schema, whitespace: bool):
        self.s, self.ws = schema, whitespace
        self._key_texts: dict[int, dict[str, str]] = {}

    def key_texts(self, node: int) -> dict[str, str]:
        """Property name -> its JSON text after the opening quote (closing quote included)."""
        kt = self._key_texts.get(node)
        if kt is None:
            kt = {name: json.dumps(name, ensure_ascii=False)[1:] for name in self.s.nodes[node].props}
            self._key_texts[node] = kt
        return kt

    # -- numbers
    def _num_ok(self, node: Node, text: str | None) -> bool:
        if text is None:
            return True
        try:
            x = int(text) if node.kind == "integer" else float(text)
        except ValueError:
            return False
        if node.minimum is not None and x < node.minimum:
            return False
        if node.maximum is not None and x > node.maximum:
            return False
        if node.multiple_of is not None:
            q = x / node.multiple_of
            if abs(q - round(q)) > 1e-9 * max(1.0, abs(q)):
                return False
        return True

    def _num_start(self, nid: int, c: str):
        node = self.s.nodes[nid]
        keep = node.minimum is not None or node.maximum is not None or node.multiple_of is not None
        if c == "-":
            if node.minimum is not None and node.minimum > 0:
                return None                       # nothing negative (nor -0) can satisfy the bound
            ph = "-"
        elif c == "0":
            ph = "0"
        elif c in "123456789":
            ph = "i"
        else:
            return None
        if keep and node.kind == "integer" and not self._int_viable(c, node.minimum, node.maximum):
            return None
        return ("num", nid, ph, c if keep else None)

    def _num_step(self, f, c: str):
        _, nid, ph, text = f
        node = self.s.nodes[nid]
        integer = node.kind == "integer"
        nxt = None
        if c in _DIGITS:
            nxt = {"-": "0" if c == "0" else "i", "i": "i", ".": "f", "f": "f", "e": "ed", "es": "ed", "ed": "ed"}.get(ph)
        elif c == "." and not integer and ph in ("0", "i"):
            nxt = "."
        elif c in "eE" and not integer and ph in ("0", "i", "f"):
            nxt = "e"
        elif c in "+-" and ph == "e":
            nxt = "es"
        if nxt is None:
            return None
        if text is not None:
            text += c
            if integer and not self._int_viable(text, node.minimum, node.maximum):
                return None
        return ("num", nid, nxt, text)

    @staticmethod
    def _int_viable(text: str, lo, hi) -> bool:
        """Can ``text`` (an integer prefix) still grow into a value inside ``[lo, hi]``?  With k more
        digits a magnitude d covers [d * 10^k, d * 10^k + 10^k - 1]; a zero takes no more digits."""
        neg = text.startswith("-")
        d = text.lstrip("-")
        if not d:
            return True
        lo = float("-inf") if lo is None else lo
        hi = float("inf") if hi is None else hi
        for k in range(0, 1 if d == "0" else 40):
            a = int(d) * 10 ** k
            b = a + 10 ** k - 1
            a, b = (-b, -a) if neg else (a, b)
            if a <= hi and b >= lo:
                return True
            if (not neg and a > hi) or (neg and b < lo):
                break                                  # more digits only move further away
        return False

    def num_complete(self, f) -> bool:
        return f[2] in _NUM_DONE and self._num_ok(self.s.nodes[f[1]], f[3])

    # -- one character
    def start(self) -> tuple:
        return (("val", self.s.root),)

    def complete(self, st: tuple) -> bool:
        return not st or (len(st) == 1 and st[0][0] == "num" and self.num_complete(st[0]))

    def step(self, st: tuple, c: str) -> list:
        """All states reachable from ``st`` by the character ``c`` (empty list: not admitted)."""
        if not st:
            return [st] if self.ws and c in _WS else []
        f, rest = st[-1], st[:-1]
        kind = f[0]
        if kind == "val":
            return self._val(rest, f[1], c)
        if kind == "lit":
            out = []
            alive = tuple(s[1:] for s in f[1] if s and s[0] == c)
            if any(s == "" for s in alive):
                out.append(rest)                              # one candidate ends here ...
            more = tuple(s for s in alive if s)
            if more:
                out.append(rest + (("lit", more),))           # ... others may go on (enum [1, 12])
            return out
        if kind == "str":
            return self._str(rest, f, c)
        if kind == "num":
            out = []
            g = self._num_step(f, c)
            if g is not None:
                out.append(rest + (g,))
            if self.num_complete(f):                          # the number ends, c belongs to the parent
                out.extend(self.step(rest, c))
            return out
        if kind == "obj":
            return self._obj(rest, f, c)
        if kind == "key":
            _, nid, seen, cands = f
            alive = tuple((name, s[1:]) for name, s in cands if s and s[0] == c)
            out = [rest + (("colon", nid, seen | {name}, name),) for name, s in alive if s == ""]
            more = tuple((name, s) for name, s in alive if s)
            if more:
                out.append(rest + (("key", nid, seen, more),))
            return out
        if kind == "colon":
            _, nid, seen, name = f
            if c == ":":
                child = self.s.nodes[nid].props[name]
                return [rest + (("obj", nid, seen, "after"), ("val", child))]
            return [st] if self.ws and c in _WS else []
        if kind == "arr":
            return self._arr(rest, f, c)
        raise AssertionError(kind)

    def _val(self, rest: tuple, nid: int, c: str) -> list:
        node = self.s.nodes[nid]
        if self.ws and c in _WS:
            return [rest + (("val", nid),)]
        k = node.kind
        if k == "union":
            out = []
            for b in node.branches:
                for s in self._val(rest, b, c):
                    if s not in out:
                        out.append(s)
            return out
        if k == "literals":
            return self.step(rest + (("lit", node.literals),), c)
        if k == "string":
            return [rest + (("str", node.min_len, node.max_len, 0, 0),)] if c == '"' else []
        if k in ("number", "integer"):
            g = self._num_start(nid, c)
            return [rest + (g,)] if g is not None else []
        if k == "object":
            return [rest + (("obj", nid, frozenset(), "open"),)] if c == "{" else []
        if k == "array":
            return [rest + (("arr", nid, 0, "open"),)] if c == "[" else []
        raise AssertionError(k)

    def _str(self, rest: tuple, f, c: str) -> list:
        _, lo, hi, n, esc = f
        if esc == 1:
            if c in '"\\/bfnrt':
                return [rest + (("str", lo, hi, n, 0),)]
            return [rest + (("str", lo, hi, n, 5),)] if c == "u" else []
        if esc > 1:
            if c not in _HEX:
                return []
            return [rest + (("str", lo, hi, n, esc - 1 if esc > 2 else 0),)]
        if c == '"':
            return [rest] if n >= lo else []
        if c < " ":
            return []                                         # raw control characters are not JSON
        if hi is not None and n >= hi:
            return []
        n2 = n + 1 if hi is not None else min(n + 1, lo)
        return [rest + (("str", lo, hi, n2, 1 if c == "\\" else 0),)]

    def _obj(self, rest: tuple, f, c: str) -> list:
        _, nid, seen, ph = f
        node = self.s.nodes[nid]
        if self.ws and c in _WS:
            return [rest + (f,)]
        left = [(name, t) for name, t in self.key_texts(nid).items() if name not in seen]
        if c == '"' and ph in ("open", "comma") and left:
            return [rest + (("key", nid, seen, tuple(left)),)]
        if c == "}" and ph in ("open", "after") and node.required <= seen:
            return [rest]
        if c == "," and ph == "after" and left:
            return [rest + (("obj", nid, seen, "comma"),)]
        return []

    def _arr(self, rest: tuple, f, c: str) -> list:
        _, nid, n, ph = f
        node = self.s.nodes[nid]
        if self.ws and c in _WS:
            return [rest + (f,)]
        if c == "]" and ph in ("open", "after") and n >= node.min_items:
            return [rest]
        if c == "," and ph == "after":
            return [rest + (("arr", nid, n, "comma"),)] if node.max_items is None or n < node.max_items else []
        if ph in ("open", "comma") and (node.max_items is None or n < node.max_items):
            # an element starts: count it (saturating, so unbounded arrays keep a finite state space)
            cap = node.max_items if node.max_items is not None else max(node.min_items, 1)
            return self._val(rest + (("arr", nid, min(n + 1, cap), "after"),), node.item, c)
        return []


_PROBE_CHARS = [chr(i) for i in range(32, 127)] + list("\t\n\r") + ["é"]


class SchemaGrammar:
    """Incremental matcher for one JSON value of a schema (the reference's ``JsonGrammar``,
    state.rs:151-200).  ``step_char`` / ``step_text`` advance it, ``valid_next_chars`` lists what
    may follow, ``is_complete`` tells whether the text so far is a whole value."""

    def __init__(self, schema, whitespace_permissive: bool = False):
        self.schema = schema if isinstance(schema, Schema) else Schema.from_json_schema(schema)
        self._m = _Machine(self.schema, whitespace_permissive)
        self.states: frozenset = frozenset([self._m.start()])
        self._memo: dict = {}          # (state set, character) -> state set; the mask walk repeats these endlessly

    def with_whitespace_permissive(self, on: bool) -> "SchemaGrammar":
        g = SchemaGrammar(self.schema, on)
        return g

    def is_whitespace_permissive(self) -> bool:
        return self._m.ws

    def reset(self) -> None:
        self.states = frozenset([self._m.start()])

    def is_complete(self) -> bool:
        return any(self._m.complete(s) for s in self.states)

    def _advance(self, states, c: str) -> frozenset:
        key = (states, c)
        hit = self._memo.get(key)
        if hit is not None:
            return hit
        out = set()
        for s in states:
            out.update(self._m.step(s, c))
        res = frozenset(out)
        if len(self._memo) > 200_000:
            self._memo.clear()
        self._memo[key] = res
        return res

    def accepts(self, text: str) -> bool:
        """Would ``text`` be admitted from the current position?  (Does not move.)"""
        st = self.states
        for c in text:
            st = self._advance(st, c)
            if not st:
                return False
        return True

    def step_char(self, c: str) -> None:
        nxt = self._advance(self.states, c)
        if not nxt:
            raise GrammarError("character %r is not admitted here" % c)
        self.states = nxt

    def step_text(self, text: str) -> None:
        st = self.states
        for i, c in enumerate(text):
            st = self._advance(st, c)
            if not st:
                raise GrammarError("character %r at offset %d is not admitted" % (c, i))
        self.states = st

    def valid_next_chars(self) -> list[str]:
        """The admitted next characters among printable ASCII, tab / newline / return, and one
        representative non-ASCII letter (``"\\u00e9"`` stands for "any other character")."""
        return [c for c in _PROBE_CHARS if self._advance(self.states, c)]


def validate(schema, text: str, whitespace_permissive: bool = True) -> bool:
    """Is ``text`` a complete value of ``schema``?"""
    g = SchemaGrammar(schema, whitespace_permissive)
    try:
        g.step_text(text)
    except GrammarError:
        return False
    return g.is_complete()


# --------------------------------------------------------------------------- tokens
class TokenMask:
    """Which token ids may come next (json_schema.rs:73-105).  ``bits`` is a bool tensor on the
    CPU; :meth:`packed` gives the reference's layout, 32 ids per little-endian word."""

    def __init__(self, bits: torch.Tensor):
        self.bits = bits

    @classmethod
    def allow_all(cls, vocab_size: int) -> "TokenMask":
        return cls(torch.ones(vocab_size, dtype=torch.bool))

    def num_allowed(self) -> int:
        return int(self.bits.sum())

    def is_allowed(self, token_id: int) -> bool:
        return 0 <= token_id < self.bits.numel() and bool(self.bits[token_id])

    def allowed_ids(self) -> list[int]:
        return self.bits.nonzero().flatten().tolist()

    def packed(self) -> torch.Tensor:
        n = self.bits.numel()
        pad = (-n) % 32
        b = torch.cat([self.bits, torch.zeros(pad, dtype=torch.bool)]).view(-1, 32).to(torch.int64)
        words = (b << torch.arange(32, dtype=torch.int64)).sum(1)
        return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        """``logits [..., V]`` with every disallowed entry set to -inf (on the logits' device)."""
        return logits.masked_fill(~self.bits.to(logits.device), float("-inf"))

    def apply_(self, logits: torch.Tensor) -> torch.Tensor:
        """In place through :func:`apply_packed_mask_` (one mask row for every logits row)."""
        return apply_packed_mask_(logits, self.packed()[None])


def unpack_mask(packed: torch.Tensor, vocab: int) -> torch.Tensor:
    """``int32 [rows, ceil(V / 32)]`` -> bool ``[rows, V]`` (bit i of word w is id ``32 w + i``)."""
    w = packed.to(torch.int64) & 0xFFFFFFFF
    bits = (w[..., None] >> torch.arange(32, device=packed.device)) & 1
    return bits.flatten(-2)[..., :vocab].bool()


def _register_token_mask_proto() -> None:
    from .. import _native

    _native.register_protos({"ft_apply_token_mask": (_native._i, [_native._vp, _native._vp, _native._ll, _native._ll,
                                                                   _native._ll, _native._i, _native._i, _native._i,
                                                                   _native._vp])})


def apply_packed_mask_(logits: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """Set ``logits[b, v] = -inf`` wherever bit v of ``packed[b]`` (or of ``packed[0]`` when it has
    one row) is clear, in place.  ``logits [rows, V]`` bf16 / fp32 with unit inner stride.  On a GPU
    this is one launch of ``ft_apply_token_mask`` (``csrc/token_mask.cu``) and the mask crosses PCIe
    as 1 bit per id; elsewhere the bits are unpacked with torch ops."""
    if logits.dim() != 2 or packed.dim() != 2 or packed.shape[0] not in (1, logits.shape[0]) or \
            packed.shape[1] != (logits.shape[1] + 31) // 32:
        raise ValueError("apply_packed_mask_: logits %s and packed mask %s do not fit" % (tuple(logits.shape), tuple(packed.shape)))
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(1) == 1:
        from .. import _native

        _register_token_mask_proto()
        m = packed.to(device=logits.device, dtype=torch.int32, non_blocking=True).contiguous()
        rc = _native.kernels().ft_apply_token_mask(logits.data_ptr(), m.data_ptr(), logits.shape[0], logits.shape[1],
                                                   logits.stride(0), m.shape[0], int(logits.dtype == torch.float32),
                                                   logits.device.index or 0, torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ft_apply_token_mask")
        return logits
    keep = unpack_mask(packed.to(logits.device), logits.shape[1])
    return logits.masked_fill_(~keep.expand_as(logits), float("-inf"))


class TokenTransitionCache:
    """Masks by matcher state (json_schema.rs:111-165): decoding revisits the same states (inside
    a string, between array elements ...), and a mask costs a walk over the vocabulary."""

    def __init__(self, max_entries: int = 4096):
        self._d: dict = {}
        self.max_entries = max_entries
        self._hits = self._misses = 0

    def __len__(self) -> int:
        return len(self._d)

    def len(self) -> int:
        """Masks held."""
        return len(self._d)

    def hits(self) -> int:
        return self._hits

    def misses(self) -> int:
        return self._misses

    def reset_counters(self) -> None:
        self._hits = self._misses = 0

    def clear(self) -> None:
        self._d.clear()

    def __len__(self) -> int:
        return len(self._d)

    def is_empty(self) -> bool:
        return not self._d

    def get(self, key, make):
        m = self._d.get(key)
        if m is not None:
            self._hits += 1
            return m
        self._misses += 1
        m = make()
        if len(self._d) >= self.max_entries:
            self._d.pop(next(iter(self._d)))
        self._d[key] = m
        return m


class _Trie:
    __slots__ = ("kids", "ids")

    def __init__(self):
        self.kids: dict = {}
        self.ids: list = []


def _build_trie(vocab: list[str], skip: set) -> _Trie:
    root = _Trie()
    for i, piece in enumerate(vocab):
        if not piece or i in skip:
            continue
        node = root
        for c in piece:
            nxt = node.kids.get(c)
            if nxt is None:
                nxt = node.kids[c] = _Trie()
            node = nxt
        node.ids.append(i)
    return root


class _NativeMasker:
    """The vocabulary trie and the walk in C++ (``csrc/host/grammar_mask.cpp``); the matcher is
    asked for a transition through a callback only the first time a (state, character) pair comes
    up.  State sets get integer ids here; one masker serves every processor of the same schema and
    vocabulary."""

    def __init__(self, grammar: "SchemaGrammar", vocab: list[str], skip: set):
        import ctypes

        import numpy as np

        from .. import _native

        lib = _native.host()
        lib.ftgm_create.restype = ctypes.c_void_p
        lib.ftgm_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        self._cb_type = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int, ctypes.c_uint)
        lib.ftgm_mask.restype = ctypes.c_longlong
        lib.ftgm_mask.argtypes = [ctypes.c_void_p, ctypes.c_int, self._cb_type, ctypes.c_void_p]
        lib.ftgm_destroy.argtypes = [ctypes.c_void_p]
        lib.ftgm_num_nodes.restype = lib.ftgm_num_transitions.restype = ctypes.c_longlong
        lib.ftgm_num_nodes.argtypes = lib.ftgm_num_transitions.argtypes = [ctypes.c_void_p]
        self._lib, self._g = lib, grammar
        offs = np.zeros(len(vocab) + 1, dtype=np.int64)
        for i, piece in enumerate(vocab):
            offs[i + 1] = offs[i] + len(piece)
        cps = np.fromiter((ord(c) for piece in vocab for c in piece), dtype=np.uint32, count=int(offs[-1]))
        skip_arr = np.zeros(len(vocab), dtype=np.uint8)
        for i in skip:
            if 0 <= i < len(vocab):
                skip_arr[i] = 1
        self._h = lib.ftgm_create(cps.ctypes.data, offs.ctypes.data, len(vocab), skip_arr.ctypes.data)
        if not self._h:
            raise RuntimeError("grammar mask: could not build the vocabulary trie")
        self.n = len(vocab)
        self._ids: dict = {}
        self._sets: list = []
        self._error: list = []

        def step(state: int, cp: int) -> int:
            try:
                nxt = grammar._advance(self._sets[state], chr(cp))
                return self.state_id(nxt) if nxt else -1
            except BaseException as e:  # noqa: BLE001   (must not propagate through the C frame)
                self._error.append(e)
                return -2

        self._cb = self._cb_type(step)

    def state_id(self, states: frozenset) -> int:
        i = self._ids.get(states)
        if i is None:
            i = self._ids[states] = len(self._sets)
            self._sets.append(states)
        return i

    def mask(self, states: frozenset) -> torch.Tensor:
        bits = torch.zeros(self.n, dtype=torch.uint8)
        rc = self._lib.ftgm_mask(self._h, self.state_id(states), self._cb, bits.data_ptr())
        if self._error:
            raise self._error.pop()
        if rc < 0:
            raise RuntimeError("grammar mask: native walk failed (%d)" % rc)
        return bits.bool()

    def stats(self) -> dict:
        return {"trie_nodes": int(self._lib.ftgm_num_nodes(self._h)), "transitions": int(self._lib.ftgm_num_transitions(self._h)),
                "states": len(self._sets)}

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.ftgm_destroy(self._h)
                self._h = None
        except Exception:  # noqa: BLE001
            pass


class JsonSchemaProcessor:
    """Token-level constrained decoding for one sequence (json_schema.rs:171-300).

    ``vocab[i]`` is the text of token ``i``.  A token is admitted iff all of its characters are
    admitted in sequence; the end-of-sequence token (``eos_token_id``) iff the value is complete;
    tokens with empty text never.  ``compute_mask`` walks the vocabulary trie with the matcher's
    state set, so a shared prefix is matched once."""

    def __init__(self, schema, vocab: list[str], eos_token_id: int | None = None,
                 whitespace_permissive: bool = False, native: bool | None = None, share: "JsonSchemaProcessor | None" = None):
        """``native``: walk the vocabulary in C++ (default: when the host library is available).
        ``share``: another processor of the same schema and vocabulary whose trie and transition
        tables this one reuses (one per batch row costs nothing extra)."""
        self.grammar_ = SchemaGrammar(schema, whitespace_permissive)
        self.vocab = list(vocab) if share is None else share.vocab
        self.eos = eos_token_id
        skip = {eos_token_id} if eos_token_id is not None else set()
        if share is not None:
            self.grammar_._memo = share.grammar_._memo          # same schema: transitions are shared too
            self._native, self._trie = share._native, share._trie
            return
        self._native, self._trie = None, None
        if native is None or native:
            try:
                self._native = _NativeMasker(self.grammar_, self.vocab, skip)
            except Exception:  # noqa: BLE001
                if native:
                    raise
        if self._native is None:
            self._trie = _build_trie(self.vocab, skip)

    @classmethod
    def from_compiled(cls, schema: Schema, vocab: list[str], **kw) -> "JsonSchemaProcessor":
        return cls(schema, vocab, **kw)

    def vocab_len(self) -> int:
        return len(self.vocab)

    def grammar(self) -> SchemaGrammar:
        return self.grammar_

    def is_complete(self) -> bool:
        return self.grammar_.is_complete()

    def reset(self) -> None:
        self.grammar_.reset()

    def _mask_for(self, states: frozenset) -> TokenMask:
        if self._native is not None:
            bits = self._native.mask(states)
            if self.eos is not None and 0 <= self.eos < len(self.vocab):
                m = self.grammar_._m
                bits[self.eos] = any(m.complete(s) for s in states)
            return TokenMask(bits)
        bits = torch.zeros(len(self.vocab), dtype=torch.bool)
        allowed: list[int] = []
        adv = self.grammar_._advance
        stack = [(self._trie, states)]
        while stack:
            node, st = stack.pop()
            for c, kid in node.kids.items():
                nxt = adv(st, c)
                if nxt:
                    if kid.ids:
                        allowed.extend(kid.ids)
                    if kid.kids:
                        stack.append((kid, nxt))
        if allowed:
            bits[torch.tensor(allowed)] = True
        if self.eos is not None and 0 <= self.eos < len(self.vocab):
            m = self.grammar_._m
            bits[self.eos] = any(m.complete(s) for s in states)
        return TokenMask(bits)

    def compute_mask(self) -> TokenMask:
        return self._mask_for(self.grammar_.states)

    def compute_mask_cached(self, cache: TokenTransitionCache) -> TokenMask:
        st = self.grammar_.states
        return cache.get(st, lambda: self._mask_for(st))

    def step_token(self, token_id: int) -> None:
        if not 0 <= token_id < len(self.vocab):
            raise GrammarError("token id %d outside the vocabulary of %d" % (token_id, len(self.vocab)))
        if token_id == self.eos:
            if not self.is_complete():
                raise GrammarError("end of sequence before the value is complete")
            return
        piece = self.vocab[token_id]
        if not piece:
            raise GrammarError("token %d has no text" % token_id)
        try:
            self.grammar_.step_text(piece)
        except GrammarError as e:
            raise GrammarError("token %d (%r): %s" % (token_id, piece, e))


class SchemaLogitsProcessor:
    """``logits_processor`` for :func:`ferrotorch_b200.models.generation.generate`: one
    :class:`JsonSchemaProcessor` per batch row, advanced by the tokens generated since the last
    call, masks shared through one :class:`TokenTransitionCache`.  The mask is built on the host
    and applied on the logits' device."""

    def __init__(self, schema, vocab: list[str], eos_token_id: int | None = None,
                 whitespace_permissive: bool = False):
        compiled = schema if isinstance(schema, Schema) else Schema.from_json_schema(schema)
        self._proto = JsonSchemaProcessor(compiled, vocab, eos_token_id, whitespace_permissive)
        self._make = lambda: JsonSchemaProcessor(compiled, vocab, eos_token_id, whitespace_permissive, share=self._proto)
        self.eos = eos_token_id
        self.cache = TokenTransitionCache()
        self.rows: list[JsonSchemaProcessor] = []
        self.fed: list[int] = []
        self.ended: list[bool] = []

    def __call__(self, generated: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        B = generated.shape[0]
        if len(self.rows) != B or any(n > generated.shape[1] for n in self.fed):
            self.rows, self.fed, self.ended = [self._make() for _ in range(B)], [0] * B, [False] * B
        masks = []
        for b in range(B):
            p = self.rows[b]
            for t in generated[b, self.fed[b]:].tolist():
                if t == self.eos:
                    self.ended[b] = True            # whatever follows an end of sequence is padding
                if not self.ended[b]:
                    p.step_token(t)
            self.fed[b] = generated.shape[1]
            if self.ended[b] and self.eos is not None:
                bits = torch.zeros(len(p.vocab), dtype=torch.bool)
                bits[self.eos] = True
                masks.append(bits)
                continue
            bits = p.compute_mask_cached(self.cache).bits
            if not bool(bits.any()) and self.eos is not None:
                # the vocabulary has no token for any admitted continuation: end the row rather
                # than sample from an empty distribution
                bits = bits.clone()
                bits[self.eos] = True
            masks.append(bits)
        return logits.masked_fill(~torch.stack(masks).to(logits.device), float("-inf"))


# --------------------------------------------------------------------------- the reference's remaining names
JsonGrammar = SchemaGrammar        # ferrotorch-grammar/src/state.rs


class PackedVocab:
    """The vocabulary as one array of code points with CSR offsets (gpu_dispatch.rs:897-956):
    ``offsets [V + 1]``, ``chars [sum of token lengths]`` (int32 tensors), ``max_token_len``."""

    def __init__(self, offsets: torch.Tensor, chars: torch.Tensor, max_token_len: int):
        self.offsets, self.chars, self.max_token_len = offsets, chars, int(max_token_len)

    @classmethod
    def pack(cls, vocab) -> "PackedVocab":
        lens = [len(t) for t in vocab]
        offsets = torch.zeros(len(lens) + 1, dtype=torch.int32)
        offsets[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0).to(torch.int32) if lens else offsets[1:]
        chars = torch.tensor([ord(c) for t in vocab for c in t], dtype=torch.int32)
        return cls(offsets, chars, max(lens, default=0))

    def __len__(self) -> int:
        return self.offsets.numel() - 1

    def token(self, i: int) -> str:
        return "".join(chr(int(c)) for c in self.chars[int(self.offsets[i]):int(self.offsets[i + 1])])

    def to(self, device) -> "PackedVocab":
        return PackedVocab(self.offsets.to(device), self.chars.to(device), self.max_token_len)


def compute_mask_gpu(processor: "JsonSchemaProcessor", packed: PackedVocab | None = None, device=None) -> TokenMask:
    """The processor's token mask with its packed words resident on ``device`` (default: the
    current CUDA device when there is one), ready for :func:`apply_packed_mask_` on device logits.
    The reference walks a compiled DFA over ``packed`` in a kernel for a few grammar states and
    falls back to the host walk for the rest (gpu_dispatch.rs ``compute_mask_gpu``); here the walk
    is always the native trie walk on the host -- transitions are memoised, so a warm mask is table
    look-ups -- and only the application of the mask runs on the GPU."""
    if packed is not None and len(packed) != processor.vocab_len():
        raise ValueError("compute_mask_gpu: packed vocabulary has %d tokens, the processor %d" % (len(packed), processor.vocab_len()))
    mask = processor.compute_mask()
    if device is None and torch.cuda.is_available():
        device = torch.device("cuda", torch.cuda.current_device())
    if device is not None:
        mask.packed_device = mask.packed().to(device, non_blocking=True)
    return mask


class BooleanEmissionStage:
    """Where a boolean literal stands while it is being emitted (state.rs:238): ``Start``, or part
    of ``true`` / ``false`` written with ``remaining`` still to come."""

    def __init__(self, kind: str, remaining: str = ""):
        self.kind, self.remaining = kind, remaining

    Start = None      # filled in below

    @classmethod
    def PartialTrue(cls, remaining: str) -> "BooleanEmissionStage":
        return cls("partial_true", remaining)

    @classmethod
    def PartialFalse(cls, remaining: str) -> "BooleanEmissionStage":
        return cls("partial_false", remaining)

    @classmethod
    def after(cls, emitted: str) -> "BooleanEmissionStage | None":
        """Stage after ``emitted`` characters of a boolean; None when they start neither literal or complete one."""
        if emitted == "":
            return cls.Start
        for word, make in (("true", cls.PartialTrue), ("false", cls.PartialFalse)):
            if word.startswith(emitted) and emitted != word:
                return make(word[len(emitted):])
        return None

    def allowed_next(self) -> str:
        return "tf" if self.kind == "start" else self.remaining[:1]

    def __eq__(self, other) -> bool:
        return isinstance(other, BooleanEmissionStage) and (self.kind, self.remaining) == (other.kind, other.remaining)

    def __hash__(self) -> int:
        return hash((self.kind, self.remaining))

    def __repr__(self) -> str:
        return "BooleanEmissionStage.Start" if self.kind == "start" else "BooleanEmissionStage(%s, remaining=%r)" % (self.kind, self.remaining)


BooleanEmissionStage.Start = BooleanEmissionStage("start")
