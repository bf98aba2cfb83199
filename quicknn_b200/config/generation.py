"""Stop ids that a model folder gives beside its config.json.

The reference collects its stop tokens from ``eos_token_id`` of config.json and, if the folder has one,
of generation_config.json as well (an integer or a list; an id outside the vocabulary is an error; the same
id is kept once; src/models/QuickNN.Models.LLM.pas:105-122,255-271).
"""
from __future__ import annotations

import json
import os
from typing import Iterable, List, Sequence


def _flatten(value) -> Iterable[int]:
    if value is None:
        return
    if isinstance(value, (list, tuple)):
        for v in value:
            yield from _flatten(v)
        return
    if isinstance(value, bool) or not isinstance(value, int):
        raise ValueError(f"a stop token must be an integer, not {value!r}")
    yield int(value)


def stop_ids_of_folder(model_dir: str, vocab_size: int, from_config: Sequence[int] = ()) -> List[int]:
    """``from_config`` (the ids of config.json, in their order) followed by the ids that
    ``generation_config.json`` of the folder adds, each id once."""
    out: List[int] = []
    for i in from_config:
        if int(i) not in out:
            out.append(int(i))
    path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(path):
        try:
            with open(path, "r", encoding="utf-8") as fh:
                data = json.load(fh)
        except (OSError, ValueError) as e:
            raise ValueError(f"invalid generation_config.json in {model_dir}: {e}") from None
        if not isinstance(data, dict):
            raise ValueError(f"invalid generation_config.json in {model_dir}: not an object")
        for i in _flatten(data.get("eos_token_id")):
            if i < 0 or i >= vocab_size:
                raise ValueError(f"generation_config.json: stop token {i} is outside the vocabulary of {vocab_size}")
            if i not in out:
                out.append(i)
    return out
