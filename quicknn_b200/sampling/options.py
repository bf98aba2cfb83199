"""Generation options, with the reference's names, defaults and validity rules.

``TLLMGenerationOptions`` (src/models/QuickNN.Models.LLM.Types.pas:29-38, defaults
:144-155): MaxNewTokens 256, HardMaxNewTokens 4096, TopK 20, AutoContinue false,
Temperature 0.6, TopP 0.95, RepetitionPenalty 1, Seed 42, EnableThinking false.
Rules (``ValidateOptions``, src/models/QuickNN.Models.LLM.pas:646-666): MaxNewTokens >= 1,
HardMaxNewTokens >= 0 and >= MaxNewTokens when AutoContinue, TopK in 1..64,
Temperature finite and >= 0, TopP in (0, 1], RepetitionPenalty finite and > 0;
thinking mode is refused for this architecture's plain chat template (:648-649).
"""
from __future__ import annotations

import dataclasses
import math
from typing import List


class OptionsError(ValueError):
    pass


@dataclasses.dataclass
class GenerationOptions:
    max_new_tokens: int = 256
    hard_max_new_tokens: int = 4096
    top_k: int = 20
    auto_continue: bool = False
    temperature: float = 0.6
    top_p: float = 0.95
    repetition_penalty: float = 1.0
    seed: int = 42
    enable_thinking: bool = False

    @classmethod
    def greedy(cls, max_new_tokens: int = 256, **kw) -> "GenerationOptions":
        return cls(max_new_tokens=max_new_tokens, temperature=0.0, **kw)

    def problems(self) -> List[str]:
        p: List[str] = []
        fin = lambda v: isinstance(v, (int, float)) and math.isfinite(v)  # noqa: E731
        if self.enable_thinking:
            p.append("enable_thinking: this chat template does not support thinking mode")
        if self.max_new_tokens < 1:
            p.append("max_new_tokens must be >= 1")
        if self.hard_max_new_tokens < 0:
            p.append("hard_max_new_tokens must be >= 0")
        if self.auto_continue and self.hard_max_new_tokens < self.max_new_tokens:
            p.append("hard_max_new_tokens must be >= max_new_tokens when auto_continue is on")
        if not (1 <= self.top_k <= 64):
            p.append("top_k must be in 1..64")
        if not fin(self.temperature) or self.temperature < 0:
            p.append("temperature must be finite and >= 0")
        if not fin(self.top_p) or not (0 < self.top_p <= 1):
            p.append("top_p must be in (0, 1]")
        if not fin(self.repetition_penalty) or self.repetition_penalty <= 0:
            p.append("repetition_penalty must be finite and > 0")
        if self.seed < 0 or self.seed >= 1 << 64:
            p.append("seed must fit 64 bits")
        return p

    def validate(self) -> None:
        p = self.problems()
        if p:
            raise OptionsError("invalid generation options: " + "; ".join(p))

    def budget(self) -> int:
        """New tokens one call may produce (``Budget``, LLM.pas:790-792)."""
        return self.hard_max_new_tokens if self.auto_continue else self.max_new_tokens


def seed_state(seed: int, index: int = 0) -> int:
    """Start state of the xorshift32 generator: low word xor high word of the 64-bit seed, 0
    replaced by 0x9E3779B9 (LLM.pas:976-978).  Sequence ``index`` of a batch uses
    ``seed + index``, so the first one draws exactly as a single request would."""
    s = (seed + index) & 0xFFFFFFFFFFFFFFFF
    x = (s & 0xFFFFFFFF) ^ (s >> 32)
    return x if x else 0x9E3779B9
