"""TifepelConfig: the typed form of a Tifepel config.json.

The design keeps its residual stream in `streams` copies (hyper-connections: a sublayer reads a learned mixture of
them through a LayerNorm without offset and writes into all of them), puts a short causal convolution (`canon.taps`)
on every sublayer's input and a learned gate on its result, and stacks two kinds of layers: attention without rotation
(query and key heads of unit root mean square, a factor on the query that grows with the logarithm of the position, a
learned bias by distance in logarithmic buckets) and Mamba-2 state-space layers.  The feed-forward routes every token
through `top` of `experts + identity` small gated experts by softmax scores plus a correction, beside a shared expert.
The embedding adds a hashed pair-of-tokens table and a learned position vector.  A span of layers may run several
times (`loop`).  Keys: `vocab`, `width`, `max_positions`, `streams`, `norm.eps`, `canon.taps`,
`embedding.bigram.{buckets, mul_prev, mul_cur}`, `layers[i].{type, mixer, mlp}`, `loop.{start, stop, times}`;
core/tifepel.cpp lists them all.

Reading, type checks and validation are the host library's (core/tifepel.cpp, TifepelConfig); this dataclass
carries the result.  Its layer records stay plain dictionaries, as config.json writes them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .. import core
from .base import ModelConfig


@dataclasses.dataclass(frozen=True)
class TifepelConfig(ModelConfig):
    architecture = "Tifepel"

    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    streams: int = 1
    embedding: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"bigram": {"buckets": 1, "mul_prev": 0, "mul_cur": 0}})
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-5})
    canon: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"taps": 1})
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    loop: Optional[Dict[str, Any]] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "TifepelConfig":
        """Type checks only; `validate` checks the sizes against one another."""
        n = core.call("global", None, "parse_config", config=raw, architecture=cls.architecture, validate=False)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in n.items() if k in names})

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        if d.get("loop") is None:
            d.pop("loop", None)
        d["architecture"] = self.architecture
        return d

    def validate(self) -> None:
        core.call("global", None, "parse_config", config=self.to_dict(), architecture=self.architecture, validate=True)
