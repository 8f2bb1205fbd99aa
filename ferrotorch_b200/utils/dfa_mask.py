"""Token masks from a finite automaton, computed for the whole vocabulary at once on any device.

For grammar states that are a finite automaton over characters (a boolean, ``null``, a fixed set of
literal values) the reference walks every token of the vocabulary through the automaton in one GPU
kernel, one thread per token (ferrotorch-cubecl/src/grammar.rs: ``kernel_compute_token_mask_dfa``
:63, ``DfaMaskInputs`` :153, ``compute_token_mask_dfa_to_gpu``; called from
ferrotorch-grammar/src/gpu_dispatch.rs).  The same walk here is a lock-step loop over character
positions with every token as one lane of a tensor: ``state = transitions[state, class(char)]`` for
``max_token_len`` steps, all on the device that holds the packed vocabulary, so on a GPU nothing but
the final mask ever has to leave it.  The conventions are the reference's:

* states ``0 .. num_states``; ``reject_state`` is a sink; a token is allowed iff its walk from
  ``start_state`` never reaches it;
* characters are mapped to classes by a 128-entry table; code points >= 128 always reject;
* an empty token is rejected (it would not advance the grammar);
* the vocabulary is packed as CSR: ``offsets [V + 1]`` into ``chars [total]``.

:func:`literal_dfa` builds the automaton for "the output so far, continued by this token, is still a
prefix of one of these literals", which covers booleans, ``null`` and string enums.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class DfaMaskInputs:
    transitions: torch.Tensor        # [num_states, num_classes] integer, next state
    char_classes: torch.Tensor       # [128] integer, class of an ASCII code point
    vocab_offsets: torch.Tensor      # [V + 1]
    vocab_chars: torch.Tensor        # [vocab_offsets[-1]] code points
    num_classes: int
    start_state: int
    reject_state: int
    max_token_len: int

    @classmethod
    def new(cls, transitions, char_classes, vocab_offsets, vocab_chars, num_classes: int, start_state: int, reject_state: int,
            max_token_len: int, vocab_size: int | None = None) -> "DfaMaskInputs | None":
        """Validated construction; ``None`` when the pieces do not fit together (offsets without
        their trailing sentinel, a table that is not ``num_states x num_classes``, states out of range)."""
        t = torch.as_tensor(transitions).long().reshape(-1)
        cc, off, ch = torch.as_tensor(char_classes).long(), torch.as_tensor(vocab_offsets).long(), torch.as_tensor(vocab_chars).long()
        if num_classes < 1 or t.numel() == 0 or t.numel() % num_classes or cc.numel() != 128 or off.numel() < 1:
            return None
        if vocab_size is not None and off.numel() != vocab_size + 1:
            return None
        n_states = t.numel() // num_classes
        if not (0 <= start_state < n_states and 0 <= reject_state < n_states):
            return None
        if int(off[-1]) != ch.numel() or (off.numel() > 1 and bool((off[1:] < off[:-1]).any())) or int(off[0]) != 0:
            return None
        if bool((t < 0).any()) or bool((t >= n_states).any()) or bool((cc < 0).any()) or bool((cc >= num_classes).any()):
            return None
        return cls(t.reshape(n_states, num_classes), cc, off, ch, int(num_classes), int(start_state), int(reject_state), int(max_token_len))

    @property
    def vocab_size(self) -> int:
        return self.vocab_offsets.numel() - 1

    def to(self, device) -> "DfaMaskInputs":
        return DfaMaskInputs(self.transitions.to(device), self.char_classes.to(device), self.vocab_offsets.to(device),
                             self.vocab_chars.to(device), self.num_classes, self.start_state, self.reject_state, self.max_token_len)

    def __repr__(self) -> str:
        return ("DfaMaskInputs(states=%d, classes=%d, vocab=%d, chars=%d, start=%d, reject=%d, max_token_len=%d)"
                % (self.transitions.shape[0], self.num_classes, self.vocab_size, self.vocab_chars.numel(), self.start_state,
                   self.reject_state, self.max_token_len))


def compute_token_mask_dfa(inputs: DfaMaskInputs, device=None) -> torch.Tensor:
    """``allow [V]`` bool on ``device`` (default: where the inputs are).  Tokens longer than
    ``max_token_len`` are walked only that far, as in the reference's bounded loop."""
    p = inputs.to(device) if device is not None else inputs
    dev = p.vocab_offsets.device
    V = p.vocab_size
    start, end = p.vocab_offsets[:-1], p.vocab_offsets[1:]
    state = torch.full((V,), p.start_state, dtype=torch.long, device=dev)
    n_chars = p.vocab_chars.numel()
    reject_class_row = p.transitions.new_full((1,), p.reject_state)
    for i in range(p.max_token_len):
        pos = start + i
        live = pos < end
        if not bool(live.any()):
            break
        ch = p.vocab_chars[pos.clamp(max=max(n_chars - 1, 0))] if n_chars else torch.zeros_like(pos)
        ascii_ = (ch >= 0) & (ch < 128)
        cls_ = p.char_classes[ch.clamp(0, 127)]
        nxt = torch.where(ascii_, p.transitions[state, cls_], reject_class_row.expand(V))
        state = torch.where(live, nxt, state)                 # the reject state maps to itself, so a rejected lane stays rejected
    return (state != p.reject_state) & (end > start)


def compute_token_mask_dfa_to_gpu(inputs: DfaMaskInputs, device="cuda") -> torch.Tensor:
    """The reference's launcher name: upload the inputs to ``device`` and walk there."""
    return compute_token_mask_dfa(inputs, device)


def literal_dfa(literals, emitted: str = "") -> tuple[torch.Tensor, torch.Tensor, int, int, int] | None:
    """Automaton for "``emitted`` + token is a prefix of one of ``literals``": returns
    ``(transitions [S, C], char_classes [128], num_classes, start_state, reject_state)`` or ``None``
    when ``emitted`` is not such a prefix itself or a literal has a non-ASCII character.  States are
    the nodes of the literals' trie plus the reject sink (state 0); classes are the distinct characters
    plus class 0 for every other character."""
    literals = [w for w in literals if w]
    if not literals or any(ord(c) >= 128 for w in literals for c in w):
        return None
    alphabet = sorted({c for w in literals for c in w})
    cls_of = {c: i + 1 for i, c in enumerate(alphabet)}
    nodes = {"": 1}
    for w in literals:
        for j in range(1, len(w) + 1):
            nodes.setdefault(w[:j], len(nodes) + 1)
    if emitted not in nodes:
        return None
    trans = torch.zeros(len(nodes) + 1, len(alphabet) + 1, dtype=torch.long)          # everything rejects ...
    for prefix, s in nodes.items():
        if prefix:
            trans[nodes[prefix[:-1]], cls_of[prefix[-1]]] = s                            # ... except the trie's edges
    classes = torch.zeros(128, dtype=torch.long)
    for c, k in cls_of.items():
        classes[ord(c)] = k
    return trans, classes, len(alphabet) + 1, nodes[emitted], 0
