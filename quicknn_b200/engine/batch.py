"""What one step brings: the tokens of a batch and where they stand."""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional

import torch


@dataclasses.dataclass
class WholeSequences:
    """The sequences of a step that goes on from cached tokens, as if each were laid out whole, cached tokens
    first: sequence b has ``start[b]`` cached tokens and brings ``new_len[b]`` rows (rows ``new_row0[b]``.. of the
    packed batch); in the whole layout it owns rows ``row0[b]`` .. ``row0[b] + length[b] - 1`` and token t of the
    packed batch is row ``tok_row[t]``.  Device arrays are int32; the counts are host integers."""

    slots: torch.Tensor             # [B]
    start: torch.Tensor             # [B]
    new_row0: torch.Tensor          # [B]
    new_len: torch.Tensor           # [B]
    row0: torch.Tensor              # [B]
    length: torch.Tensor            # [B] = start + new_len
    tok_row: torch.Tensor           # [T]
    total: int                      # rows of the whole layout
    longest: int                    # longest whole sequence
    most_new: int                   # most rows that one sequence brings


@dataclasses.dataclass
class StepBatch:
    """Device-side description of one step.

    ``mode`` is "prefill" when every sequence starts at its first token (the whole
    prompts, packed one after another), "decode" when every sequence goes on by
    one token, and "extend" for everything else (sequences that go on by several
    tokens, or some that start beside others that go on).  Row t of the packed batch
    belongs to the sequence in slot ``tok_slot[t]`` (a negative slot marks a padding
    row: nothing is written for it and it attends to nothing) at position
    ``tok_pos[t]``; its sequence's first row is ``tok_row0[t]``.

    ``max_seq`` (the longest sequence the cache was built for) and ``tuning`` (options
    that the engine's owner set and that parts may look up by name, for instance
    ``decode_splits``) let a part choose its schedule; ``scratch`` is the scratch
    memory that the parts asked for with ``scratch_need`` (bytes; None if none did).
    ``longest`` and ``spread`` describe the lengths of a decode step's sequences in coarse
    classes (an upper bound of the longest sequence; a typical ratio of the longest to the
    mean), 0 when unknown: a schedule that a part derives from them holds for every step
    of the same classes, which is what the engine captures a decode graph for.
    """

    mode: str
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor            # [T] int32
    tok_pos: torch.Tensor           # [T] int32
    tok_slot: torch.Tensor          # [T] int32
    tok_row0: torch.Tensor          # [T] int32
    slots: torch.Tensor             # [B] int32
    want_rows: torch.Tensor         # [R] int32: rows whose logits are returned
    act_dtype: torch.dtype
    max_q_len: int = 1              # longest run of tokens that one sequence brings
    seq_row0: Optional[torch.Tensor] = None   # [B] int32: first row of each sequence in the packed batch
    seq_len: Optional[torch.Tensor] = None    # [B] int32: tokens that each sequence brings
    max_seq: int = 0
    tuning: Mapping[str, Any] = dataclasses.field(default_factory=dict)
    scratch: Optional[torch.Tensor] = None    # uint8
    want_every_row: bool = False              # want_rows is 0, 1, ..., T-1: no gather is needed
    whole: Optional[WholeSequences] = None    # extend steps: the sequences with their cached tokens in front
    longest: int = 0                          # decode: class of the longest sequence (an upper bound), 0 = unknown
    spread: float = 0.0                       # decode: class of longest / mean length (1.0, 1.25, 1.6 or 2.2), 0 = unknown
