"""Sampling parameters, request and result types, with the reference's names and meanings
(src/engine/types.h:16-25, 56-96) and a model folder's defaults
(generation_config.json, src/models/config_util.cpp:162-182)."""
from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from typing import Callable, List, Optional

from ..config.json_util import get_bool_or, get_int_list, read_json


@dataclass
class SamplingParams:
    temperature: float = 1.0          # 0 = greedy
    top_k: int = 0                    # 0 = off
    top_p: float = 1.0                # 1 = off
    min_p: float = 0.0                # 0 = off
    repetition_penalty: float = 1.0   # 1 = off; applied to tokens of prompt + output
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None        # None: a fresh random seed per request

    def greedy(self) -> bool:
        """src/engine/sampler.h:36."""
        return self.temperature <= 0.0 or self.top_k == 1

    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0)

    def needs_logits(self) -> bool:
        """False when the largest logit's index is the answer whatever the history
        (src/engine/sampler.h:28-31)."""
        return not self.greedy() or self.has_penalties()

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive")


@dataclass
class GenerateRequest:
    prompt: List[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    max_new_tokens: int = 512
    stop_token_ids: List[int] = field(default_factory=list)   # ends generation; not returned


FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED, FINISH_ERROR = "stop", "length", "cancelled", "error"


@dataclass
class GenerateStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0     # between the first and the last emitted token
    batch_size: int = 1

    def prefill_tok_per_s(self) -> float:
        return self.prompt_tokens * 1000.0 / self.prefill_ms if self.prefill_ms > 0 else 0.0

    def decode_tok_per_s(self) -> float:
        """The first token belongs to the prefill (src/engine/types.h:84-86)."""
        if self.decode_ms > 0 and self.generated_tokens > 1:
            return (self.generated_tokens - 1) * 1000.0 / self.decode_ms
        return 0.0


@dataclass
class GenerateResult:
    finish: str = FINISH_STOP
    tokens: List[int] = field(default_factory=list)   # generated tokens, stop token excluded
    stats: GenerateStats = field(default_factory=GenerateStats)
    error: str = ""


# Called for every generated token as (request index, token); returning False cancels that request.
TokenCallback = Callable[[int, int], bool]


def read_generation_defaults(folder: str):
    """(SamplingParams, stop ids) from generation_config.json. Without the file the defaults stand
    (temperature 1); with it, do_sample false means greedy (src/models/config_util.cpp:162-182)."""
    p = SamplingParams()
    path = os.path.join(folder, "generation_config.json")
    if not os.path.isfile(path):
        return p, []
    j = read_json(path)
    where = "generation_config.json"
    if not get_bool_or(j, "do_sample", False, where):
        p = replace(p, temperature=0.0)
    elif isinstance(j.get("temperature"), (int, float)) and not isinstance(j.get("temperature"), bool):
        p = replace(p, temperature=float(j["temperature"]))
    if isinstance(j.get("top_k"), int) and not isinstance(j.get("top_k"), bool):
        p = replace(p, top_k=j["top_k"])
    for key in ("top_p", "min_p", "repetition_penalty"):
        v = j.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            p = replace(p, **{key: float(v)})
    return p, get_int_list(j, "eos_token_id", where)


def merged_stop_ids(folder: str, config=None) -> List[int]:
    """The ids that end a sequence: generation_config.json's `eos_token_id` and config.json's, merged, sorted,
    each once (src/models/lfm3/lfm3_model.cpp:69-77; the reference adds the tokenizer's end-of-turn id, and
    refuses a model without any: a folder of random weights may have none here). `config`: the typed
    configuration, whose `eos_token_id` holds config.json's."""
    _, gen_stops = read_generation_defaults(folder)
    cfg_stops = list(getattr(config, "eos_token_id", ()) or ())
    return sorted(set(gen_stops) | set(cfg_stops))
