"""The cache: a slot per sequence, keys and values per cache line, fixed-size state.

Layout, ours (the reference keeps one sequence, one fp32 tensor per layer with
K transposed ``[nkv][hd][C]`` and V ``[nkv][C][hd]`` at full capacity on every layer,
src/models/QuickNN.Models.Gemma2.pas:97,125 and shaders/tensor.comp:312-317, and
the window only limits reads, shaders/attention.comp:24):

* cache lines with the same need (kv heads, head size, window) form a *group*
  with storage of its own: K and V pools ``[line][page][kv head][PAGE][head_dim]``
  of PAGE = 64 positions, and one page table ``[slot][page index]`` for the group
  (all lines of a group fill in step, so they share page ids);
* a group with a window keeps a ring of ``ceil(window / PAGE) * PAGE`` positions
  per sequence: position p lives at ring index ``p mod ring``;
* sizes are in tokens: ``max_tokens`` is the most tokens that live sequences hold
  at one time, each rounded up to a whole page;
* fixed-size state per (state line, slot), zeroed when the slot is handed out,
  never rewound (the reference keeps such state inside its recurrent models and
  resets it on a prefix mismatch, src/models/QuickNN.Models.LLM.pas:723-731).
  Gemma 2 asks for none, so the region has zero lines there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed
from .pages import PAGE, CacheFull, PagePool, SlotTable
from .upload import PinnedUploader

def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclasses.dataclass
class LineView:
    """What a mixer sees of its cache line."""

    k: torch.Tensor                 # [pages, kv heads, PAGE, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor        # [slots, pages per sequence] int32 (device)
    ring: int                       # 0 = every position kept
    page_size: int
    slot_len: torch.Tensor          # [slots] int32 (device): length after the running step
    state: Optional[torch.Tensor]   # [slots, *shape] or None
    writes: bool = True


class CacheGroup:
    def __init__(self, need: CacheNeed, lines: List[int], n_pages: int, max_slots: int, max_seq: int,
                 dtype: torch.dtype, device):
        self.need = need
        self.lines = lines
        if need.window is not None and need.window < max_seq:
            self.ring = _round_up(need.window, PAGE)
            self.pages_per_seq = self.ring // PAGE
        else:
            self.ring = 0
            self.pages_per_seq = _round_up(max_seq, PAGE) // PAGE
        self.pool = PagePool(n_pages)
        shape = (len(lines), n_pages, need.n_kv_heads, PAGE, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_host = np.zeros((max_slots, self.pages_per_seq), dtype=np.int32)
        self.table_dev = torch.zeros((max_slots, self.pages_per_seq), dtype=torch.int32, device=device)
        self.held: List[List[int]] = [[] for _ in range(max_slots)]
        self.dirty: set = set()

    def pages_for(self, length: int) -> int:
        return min(_round_up(length, PAGE) // PAGE, self.pages_per_seq)

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class KVCache:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], states: Sequence[Optional[StateNeed]],
                 max_tokens: int, max_slots: int, max_seq: int, dtype: torch.dtype, device):
        if max_tokens < 1 or max_slots < 1 or max_seq < 1:
            raise ValueError("max_tokens, max_slots and max_seq must be positive")
        self.dtype, self.device = dtype, device
        self.max_tokens = _round_up(max_tokens, PAGE)
        self.max_slots, self.max_seq = max_slots, max_seq
        self.slots = SlotTable(max_slots)
        n_pages = self.max_tokens // PAGE + 1          # + page 0
        self.groups: List[CacheGroup] = []
        self._line_group: Dict[int, Tuple[int, int]] = {}
        by_key: Dict[Tuple, List[int]] = {}
        for line, need in enumerate(needs):
            if need is not None:
                by_key.setdefault(need.group_key(), []).append(line)
        for key, lines in by_key.items():
            # a sequence of a windowed group never holds more than its ring, so that group's pool
            # needs no more than a ring per slot however many tokens the other groups keep
            w = needs[lines[0]].window
            mine = n_pages
            if w is not None and w < max_seq:
                mine = min(n_pages, max_slots * (_round_up(w, PAGE) // PAGE) + 1)
            g = CacheGroup(needs[lines[0]], lines, mine, max_slots, max_seq, dtype, device)
            for i, line in enumerate(lines):
                self._line_group[line] = (len(self.groups), i)
            self.groups.append(g)
        self.uploader = PinnedUploader(device, entries=32)
        self.lengths_host = np.zeros(max_slots, dtype=np.int32)
        self.longest_host = np.zeros(max_slots, dtype=np.int32)    # the longest that a slot's sequence has been: what its rings have overwritten
        self.lengths_dev = torch.zeros(max_slots, dtype=torch.int32, device=device)
        self._lengths_dirty = False
        self.state: Dict[int, torch.Tensor] = {}
        for line, st in enumerate(states):
            if st is not None:
                sd = dtype if st.dtype == "compute" else getattr(torch, st.dtype)
                self.state[line] = torch.zeros((max_slots,) + tuple(st.shape), dtype=sd, device=device)

    # ---- slots ------------------------------------------------------------------------
    def allocate(self) -> int:
        slot = self.slots.take()
        self.lengths_host[slot] = 0
        self.longest_host[slot] = 0
        self._lengths_dirty = True
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        self.slots.give_back(slot)                      # raises on a double free
        for g in self.groups:
            g.pool.give_back(g.held[slot])
            g.held[slot] = []
            g.table_host[slot, :] = 0
            g.dirty.add(slot)
        self.lengths_host[slot] = 0
        self.longest_host[slot] = 0
        self._lengths_dirty = True

    def length(self, slot: int) -> int:
        return int(self.lengths_host[slot])

    def tokens_held(self) -> int:
        """Tokens that live sequences hold, each rounded up to a whole page."""
        return sum(_round_up(int(self.lengths_host[s]), PAGE) for s in self.slots.live())

    def extend(self, slot_lengths: Sequence[Tuple[int, int]]) -> None:
        """Grow sequences to new lengths: ``[(slot, new_length), ...]``.  Either all fit or
        nothing changes."""
        want: List[List[Tuple[int, int]]] = [[] for _ in self.groups]
        for slot, new_len in slot_lengths:
            if not self.slots.is_live(slot):
                raise RuntimeError(f"slot {slot} is not in use")
            if new_len < self.lengths_host[slot]:
                raise ValueError(f"slot {slot}: a sequence cannot shrink ({self.lengths_host[slot]} -> {new_len})")
            if new_len > self.max_seq:
                raise CacheFull(f"slot {slot}: {new_len} tokens exceed the longest sequence "
                                f"the cache was built for ({self.max_seq})")
            for gi, g in enumerate(self.groups):
                extra = g.pages_for(new_len) - len(g.held[slot])
                if extra > 0:
                    want[gi].append((slot, extra))
        for gi, g in enumerate(self.groups):
            total = sum(e for _, e in want[gi])
            if total > g.pool.n_free:
                raise CacheFull(f"the cache holds at most {self.max_tokens} tokens "
                                f"({g.pool.n_free} free pages of {PAGE}, {total} needed)")
        for gi, g in enumerate(self.groups):
            for slot, extra in want[gi]:
                start = len(g.held[slot])
                pages = g.pool.take(extra)
                g.held[slot].extend(pages)
                g.table_host[slot, start:start + extra] = pages
                g.dirty.add(slot)
        for slot, new_len in slot_lengths:
            self.lengths_host[slot] = new_len
            self.longest_host[slot] = max(int(self.longest_host[slot]), new_len)
        self._lengths_dirty = True

    def truncate(self, slot_lengths: Sequence[Tuple[int, int]]) -> None:
        """Shorten sequences to earlier lengths and give back the pages beyond them: the undo of
        an ``extend`` whose step could not be launched.  Cells beyond the new length keep whatever
        was written; nothing reads them."""
        for slot, new_len in slot_lengths:
            if not self.slots.is_live(slot):
                continue
            if new_len > self.lengths_host[slot]:
                raise ValueError(f"slot {slot}: truncate cannot grow a sequence")
            for g in self.groups:
                keep = g.pages_for(new_len)
                if keep < len(g.held[slot]):
                    g.pool.give_back(g.held[slot][keep:])
                    g.table_host[slot, keep:] = 0
                    del g.held[slot][keep:]
                    g.dirty.add(slot)
            self.lengths_host[slot] = new_len
        self._lengths_dirty = True

    def rewind_limit(self, slot: int) -> int:
        """The shortest length that ``truncate`` may bring the sequence in ``slot`` to with everything still
        there that the next token needs: any length for groups that keep every position; for a ring the
        positions that later tokens have overwritten are gone, so a sequence that has been L tokens long can go
        back to ``L - (ring - window + 1)`` at most; fixed-size state describes the whole sequence and cannot go back at all
        (the reference rebuilds recurrent state on a changed prefix, src/models/QuickNN.Models.LLM.pas:725-733)."""
        length, longest = int(self.lengths_host[slot]), int(self.longest_host[slot])
        if self.state:
            return length
        limit = 0
        for g in self.groups:
            if g.ring and longest > g.ring:
                limit = max(limit, longest - (g.ring - int(g.need.window) + 1))
        return max(0, min(limit, length))

    def sync(self) -> None:
        """Bring the device copies of the page tables and lengths up to date."""
        for g in self.groups:
            if g.dirty:
                rows = sorted(g.dirty)
                if len(rows) > 8:
                    self.uploader.send(g.table_dev, g.table_host)
                else:
                    for r in rows:
                        self.uploader.send(g.table_dev[r], g.table_host[r])
                g.dirty.clear()
        if self._lengths_dirty:
            self.uploader.send(self.lengths_dev, self.lengths_host)
            self._lengths_dirty = False

    # ---- views ------------------------------------------------------------------------
    def line(self, line: int, writes: bool = True) -> Optional[LineView]:
        st = self.state.get(line)
        if line not in self._line_group:
            if st is None:
                return None
            return LineView(None, None, None, 0, PAGE, self.lengths_dev, st, writes)
        gi, li = self._line_group[line]
        g = self.groups[gi]
        return LineView(g.k[li], g.v[li], g.table_dev, g.ring, PAGE, self.lengths_dev, st, writes)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(t.numel() * t.element_size() for t in self.state.values())

    def bytes_read_per_step(self, slots: Sequence[int]) -> int:
        """Bytes of keys and values that one decode step of these sequences has to read."""
        total = 0
        for g in self.groups:
            per_tok = 2 * g.need.n_kv_heads * g.need.head_dim * g.k.element_size() * len(g.lines)
            for s in slots:
                n = int(self.lengths_host[s])
                if g.need.window is not None:
                    n = min(n, g.need.window)
                total += n * per_tok
        return total

    def verify_device(self) -> None:
        """The device copies of the page tables and lengths are what the host holds (after ``sync``, with the
        copies complete: this waits for the device).  A check for tests and for hunting a fault: a page table that
        reached the device late or from a reused staging buffer shows here, not as a wrong token somewhere."""
        self.sync()
        if torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)
        for i, g in enumerate(self.groups):
            if not np.array_equal(g.table_dev.cpu().numpy(), g.table_host):
                bad = np.argwhere(g.table_dev.cpu().numpy() != g.table_host)[0]
                raise AssertionError(f"group {i}: page table on the device differs at slot {bad[0]}, entry {bad[1]}")
        if not np.array_equal(self.lengths_dev.cpu().numpy(), self.lengths_host):
            raise AssertionError("the lengths on the device differ from the host's")

    def audit(self) -> None:
        """No page lost, held twice or freed twice; tables agree with what slots hold."""
        for g in self.groups:
            g.pool.audit()
            seen = set()
            for slot, pages in enumerate(g.held):
                if pages and not self.slots.is_live(slot):
                    raise AssertionError(f"free slot {slot} still holds pages")
                for i, p in enumerate(pages):
                    if p in seen:
                        raise AssertionError(f"page {p} is held twice")
                    seen.add(p)
                    if g.table_host[slot, i] != p:
                        raise AssertionError(f"page table of slot {slot} disagrees with its pages")
                if len(pages) != g.pages_for(int(self.lengths_host[slot])) and self.slots.is_live(slot):
                    raise AssertionError(f"slot {slot} holds {len(pages)} pages for "
                                         f"{self.lengths_host[slot]} tokens")
            if len(seen) != g.pool.n_held:
                raise AssertionError("the pool counts pages that no slot holds")
