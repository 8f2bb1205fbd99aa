"""Paged KV cache: host-side page bookkeeping + device-side storage consumed by kernels.

Bookkeeping mirrors the reference (ferrotorch-nn/src/paged_attention.rs:155-532): a
``PagePool`` with O(1) allocate / free, a per-sequence page list, and a manager that adds,
extends and drops sequences.  Unlike the reference, the pages are device memory
(``[num_blocks, block_size, n_kv_heads, head_dim]`` for K and for V, per layer) and the block
table is a device tensor read by ``ft_kv_append`` / ``ft_paged_decode`` (``csrc/paged_attn.cu``).
"""
from __future__ import annotations

import torch

from .. import _native
from ..ops import functional as F

_i, _ll, _f, _vp = _native._i, _native._ll, _native._f, _native._vp
_native.register_protos({
    "ft_kv_append": (_i, [_vp] * 7 + [_i, _i, _i, _i, _ll, _ll, _i, _i, _i, _i, _vp]),
    "ft_paged_decode_scratch": (_ll, [_i, _i, _i, _i]),
    "ft_paged_decode": (_i, [_vp] * 7 + [_i, _i, _i, _i, _ll, _ll, _i, _i, _i, _f, _i, _i, _vp]),
})


class OutOfPages(RuntimeError):
    pass


class PagePool:
    """Free-list of page ids (paged_attention.rs:155-260) with a reference count per page: a page that several
    sequences share (a common prompt prefix) returns to the free list when its last holder lets go."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._refs = [0] * num_pages

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("page pool exhausted (%d pages)" % self.num_pages)
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def retain(self, page: int) -> int:
        """One more holder of an allocated page."""
        if not 0 <= page < self.num_pages or self._refs[page] == 0:
            raise ValueError("page %d is not allocated" % page)
        self._refs[page] += 1
        return page

    def ref_count(self, page: int) -> int:
        return self._refs[page]

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError("page %d out of range" % page)
        if self._refs[page] == 0:
            raise ValueError("page %d is free already" % page)
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def alloc_page(self):
        """A free page id, or ``None`` when the pool is exhausted (paged_attention.rs:200; ``allocate`` raises)."""
        return self.allocate() if self._free else None

    free_page = free

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    @property
    def num_total(self) -> int:
        return self.num_pages


class PagedKVCache:
    """Block tables for up to ``max_seqs`` sequences over one :class:`PagePool`, plus the device
    K/V pages of every layer.  ``block_size`` tokens per page (16 in the benchmark configs)."""

    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, num_blocks: int, max_seqs: int,
                 max_seq_len: int, block_size: int = 16, device="cuda", dtype=torch.bfloat16):
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        self.block_size, self.num_blocks, self.max_seqs = block_size, num_blocks, max_seqs
        self.max_blocks = (max_seq_len + block_size - 1) // block_size
        self.device = torch.device(device)
        self.pool = PagePool(num_blocks)
        shape = (num_blocks, block_size, n_kv_heads, head_dim)
        self.k = [torch.zeros(shape, device=self.device, dtype=dtype) for _ in range(n_layers)]
        self.v = [torch.zeros(shape, device=self.device, dtype=dtype) for _ in range(n_layers)]
        self._table_host = torch.full((max_seqs, self.max_blocks), -1, dtype=torch.int32)
        self.block_table = self._table_host.to(self.device)
        self._pages: list[list[int]] = [[] for _ in range(max_seqs)]
        self.lengths = [0] * max_seqs
        self._dirty = False

    # ------------------------------------------------------------------ bookkeeping (host)
    def reserve(self, seq: int, new_len: int) -> None:
        """Make sure sequence ``seq`` has pages for ``new_len`` tokens."""
        need = (new_len + self.block_size - 1) // self.block_size
        if need > self.max_blocks:
            raise ValueError("sequence length %d exceeds max_seq_len" % new_len)
        pages = self._pages[seq]
        while len(pages) < need:
            p = self.pool.allocate()
            self._table_host[seq, len(pages)] = p
            pages.append(p)
            self._dirty = True
        self.lengths[seq] = max(self.lengths[seq], new_len)

    def adopt(self, seq: int, pages: list, length: int) -> None:
        """Start sequence ``seq`` on pages that already hold its first ``length`` tokens (whole pages that
        another sequence filled; every one gains a holder).  The sequence must be empty."""
        if self._pages[seq]:
            raise ValueError("adopt: sequence %d already has pages" % seq)
        if length != len(pages) * self.block_size or len(pages) > self.max_blocks:
            raise ValueError("adopt: %d pages of %d tokens cannot hold a prefix of %d" % (len(pages), self.block_size, length))
        for i, p in enumerate(pages):
            self._table_host[seq, i] = self.pool.retain(p)
        self._pages[seq] = list(pages)
        self.lengths[seq] = length
        self._dirty = bool(pages) or self._dirty

    def pages_of(self, seq: int) -> list:
        return list(self._pages[seq])

    def free_sequence(self, seq: int) -> None:
        for p in self._pages[seq]:
            self.pool.free(p)
        self._pages[seq] = []
        self._table_host[seq].fill_(-1)
        self.lengths[seq] = 0
        self._dirty = True

    def sync_table(self) -> torch.Tensor:
        if self._dirty:
            self.block_table.copy_(self._table_host, non_blocking=True)
            self._dirty = False
        return self.block_table

    # ------------------------------------------------------------------ device ops
    def append(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, positions: torch.Tensor,
               seq_ids: torch.Tensor | None = None, tokens_per_seq: int = 1) -> None:
        """Write ``k_new / v_new [T, Hkv, D]`` at ``positions [T]`` (int32).  Token i belongs to
        sequence ``seq_ids[i]`` or ``i // tokens_per_seq``.  Pages must have been reserved."""
        T = k_new.shape[0]
        table = self.sync_table()
        if not k_new.is_cuda:
            sid = (seq_ids if seq_ids is not None else torch.arange(T) // tokens_per_seq).long()
            pos = positions.long()
            blk = self._table_host[sid, pos // self.block_size].long()
            if bool((blk < 0).any()):
                raise ValueError("PagedKVCache.append: a position has no page (reserve the sequence first)")
            self.k[layer][blk, pos % self.block_size] = k_new.to(self.k[layer].dtype)
            self.v[layer][blk, pos % self.block_size] = v_new.to(self.v[layer].dtype)
            return
        ldk = k_new.stride(0)
        ldv = v_new.stride(0)
        rc = _native.kernels().ft_kv_append(
            k_new.data_ptr(), v_new.data_ptr(), self.k[layer].data_ptr(), self.v[layer].data_ptr(),
            table.data_ptr(), positions.data_ptr(), seq_ids.data_ptr() if seq_ids is not None else None, T,
            tokens_per_seq, self.n_kv_heads, self.head_dim, ldk, ldv, self.block_size, self.max_blocks,
            self.num_blocks, F._dev(k_new), F._stream())
        _native.check(rc, "ft_kv_append")

    def decode(self, layer: int, q: torch.Tensor, ctx_len: torch.Tensor, scale: float | None = None,
               n_splits: int = 0, seq_ids: torch.Tensor | None = None) -> torch.Tensor:
        """One query token per sequence: ``q [B, Hq, D]``, ``ctx_len [B]`` int32 -> ``[B, Hq, D]``.  Row b
        reads sequence b, or sequence ``seq_ids[b]`` (a batch of any subset of the live sequences: the rows of
        the block table are gathered in that order)."""
        B, Hq, D = q.shape
        scale = scale if scale is not None else D ** -0.5
        table = self.sync_table()
        if not q.is_cuda:
            return self._decode_reference(layer, q, ctx_len, scale, seq_ids)
        if seq_ids is not None:
            table = table.index_select(0, seq_ids.to(device=table.device, dtype=torch.long)).contiguous()
        lib = _native.kernels()
        if n_splits <= 0:
            ctas = B * self.n_kv_heads
            n_splits = 1 if ctas >= 256 else max(1, min(8, 296 // max(ctas, 1)))
        out = torch.empty(q.shape, device=q.device, dtype=q.dtype)
        n_scr = int(lib.ft_paged_decode_scratch(B, Hq, D, n_splits))
        scratch = F._get_scratch("paged_decode", n_scr, q.device) if n_scr else None
        rc = lib.ft_paged_decode(q.data_ptr(), self.k[layer].data_ptr(), self.v[layer].data_ptr(), table.data_ptr(),
                                 ctx_len.data_ptr(), out.data_ptr(), scratch.data_ptr() if scratch is not None else None,
                                 B, Hq, self.n_kv_heads, D, q.stride(0), out.stride(0), self.block_size,
                                 self.max_blocks, self.num_blocks, float(scale), n_splits, F._dev(q), F._stream())
        _native.check(rc, "ft_paged_decode")
        return out

    def gather(self, layer: int, seq: int, length: int):
        """Contiguous ``[length, Hkv, D]`` K and V of one sequence (debug / reference path;
        paged_attention.rs ``get_keys`` / ``get_values``)."""
        pages = self._pages[seq][: (length + self.block_size - 1) // self.block_size]
        idx = torch.tensor(pages, device=self.k[layer].device, dtype=torch.long)
        k = self.k[layer][idx].reshape(-1, self.n_kv_heads, self.head_dim)[:length]
        v = self.v[layer][idx].reshape(-1, self.n_kv_heads, self.head_dim)[:length]
        return k, v

    # ---- accessors under the reference's names (paged_attention.rs:359-395; there one object per
    # sequence, here one per model, hence the ``seq`` argument)
    def get_keys(self, seq: int, layer: int = 0) -> torch.Tensor:
        return self.gather(layer, seq, self.lengths[seq])[0]

    def get_values(self, seq: int, layer: int = 0) -> torch.Tensor:
        return self.gather(layer, seq, self.lengths[seq])[1]

    def len(self, seq: int | None = None) -> int:
        """Tokens of one sequence, or of all sequences together."""
        return self.lengths[seq] if seq is not None else sum(self.lengths)

    def is_empty(self, seq: int | None = None) -> bool:
        return self.len(seq) == 0

    def num_pages(self, seq: int | None = None) -> int:
        """Pages held by one sequence, or by all of them."""
        return len(self._pages[seq]) if seq is not None else self.pool.num_used

    def free_all(self) -> None:
        for s in range(self.max_seqs):
            if self._pages[s]:
                self.free_sequence(s)

    def _decode_reference(self, layer, q, ctx_len, scale, seq_ids=None):
        """Host form of the paged-decode kernel, all rows at once: the pages of every row are gathered through
        the block table into a padded ``[B, L, Hkv, D]`` view and positions past a row's length are masked."""
        B, Hq, D = q.shape
        rows = torch.arange(B) if seq_ids is None else seq_ids.long().cpu()
        ctx = ctx_len.long().cpu()
        n_blk = int((int(ctx.max()) + self.block_size - 1) // self.block_size)
        pages = self._table_host[rows, :n_blk].long().clamp_(min=0)          # unreserved slots read page 0 and are masked
        k = self.k[layer][pages].reshape(B, n_blk * self.block_size, self.n_kv_heads, D).float()
        v = self.v[layer][pages].reshape(B, n_blk * self.block_size, self.n_kv_heads, D).float()
        g = Hq // self.n_kv_heads
        qf = q.float().reshape(B, self.n_kv_heads, g, D)
        s = torch.einsum("bhgd,blhd->bhgl", qf, k) * scale
        dead = torch.arange(n_blk * self.block_size)[None] >= ctx[:, None]
        s = s.masked_fill(dead[:, None, None, :], float("-inf"))
        o = torch.einsum("bhgl,blhd->bhgd", torch.softmax(s, -1), v)
        return o.reshape(B, Hq, D).to(q.dtype)


class PagedAttentionManager:
    """Multi-sequence front end: hands out sequence slots, grows and frees them
    (paged_attention.rs:447-532)."""

    def __init__(self, cache: PagedKVCache):
        self.cache = cache
        self._free_slots = list(range(cache.max_seqs - 1, -1, -1))
        self.active: dict[int, int] = {}
        self._filled: dict[int, dict[int, int]] = {}        # tokens written through append_kv, per sequence and layer

    def add_sequence(self, prompt_len: int = 0) -> int:
        if not self._free_slots:
            raise OutOfPages("no free sequence slot")
        s = self._free_slots.pop()
        try:
            self.cache.reserve(s, prompt_len)
        except OutOfPages:
            self.cache.free_sequence(s)
            self._free_slots.append(s)
            raise
        self.active[s] = prompt_len
        return s

    def extend(self, seq: int, n_tokens: int = 1) -> int:
        new_len = self.active[seq] + n_tokens
        self.cache.reserve(seq, new_len)
        self.active[seq] = new_len
        return new_len

    def remove_sequence(self, seq: int) -> None:
        self.cache.free_sequence(seq)
        del self.active[seq]
        self._filled.pop(seq, None)
        self._free_slots.append(seq)
        self._free_slots.sort(reverse=True)  # lowest free slot is handed out first

    @property
    def free_pages(self) -> int:
        return self.cache.pool.num_free

    def num_sequences(self) -> int:
        return len(self.active)

    def pool_utilization(self) -> float:
        """Fraction of the pages in use, 0.0 .. 1.0 (paged_attention.rs:525)."""
        pool = self.cache.pool
        return pool.num_used / pool.num_total if pool.num_total else 0.0

    def pool(self) -> PagePool:
        return self.cache.pool

    # ---- the reference's data-carrying calls (paged_attention.rs:485-510): its manager owns one
    # cache per sequence; here one paged cache serves every layer, hence the ``layer`` argument
    def append_kv(self, seq_id: int, key: torch.Tensor, value: torch.Tensor, layer: int = 0) -> None:
        """Append ``key`` / ``value`` (``[new_tokens, num_kv_heads, head_dim]``, or flat with that many
        elements) to sequence ``seq_id``.  Layer 0 grows the sequence (pages are taken from the pool as
        needed); other layers write the same positions, so append layer 0 first."""
        if seq_id not in self.active:
            raise ValueError("PagedAttentionManager: invalid sequence id %d" % seq_id)
        c = self.cache
        key, value = key.reshape(-1, c.n_kv_heads, c.head_dim), value.reshape(-1, c.n_kv_heads, c.head_dim)
        if key.shape != value.shape:
            raise ValueError("append_kv: key %s and value %s differ" % (tuple(key.shape), tuple(value.shape)))
        n = key.shape[0]
        filled = self._filled.setdefault(seq_id, {})
        start = filled.get(layer, 0)
        if start + n > self.active[seq_id]:
            self.extend(seq_id, start + n - self.active[seq_id])
        dev = c.k[layer].device
        pos = torch.arange(start, start + n, dtype=torch.int32, device=dev)
        sid = torch.full((n,), seq_id, dtype=torch.int32, device=dev)
        c.append(layer, key.to(device=dev, dtype=c.k[layer].dtype), value.to(device=dev, dtype=c.v[layer].dtype), pos, sid)
        filled[layer] = start + n

    def get_kv(self, seq_id: int, layer: int = 0):
        """``(keys, values)`` of a sequence as contiguous ``[tokens, num_kv_heads, head_dim]`` tensors."""
        if seq_id not in self.active:
            raise ValueError("PagedAttentionManager: invalid sequence id %d" % seq_id)
        return self.cache.gather(layer, seq_id, self._filled.get(seq_id, {}).get(layer, self.active[seq_id]))
