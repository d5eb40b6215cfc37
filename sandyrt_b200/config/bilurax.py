"""BiluraxConfig: the typed form of a Bilurax config.json.

The design stacks pre-norm layers whose attention has no positions in its scores: a token shift on the mixer's
input, biases, an RMS norm over the whole query row and the whole key row, values of unit root mean square per head, a
learned temperature per head, scores pressed through `softcap * tanh(score / softcap)`, and chunks of `mask.size`
positions (a query sees the keys of its own chunk).  The feed-forward is dense (`relu(up h)^2`), a mixture of small
gated experts chosen by sigmoid scores plus a correction inside the best groups of experts, or absent.  A span of
layers may run several times (`loop`), the embedding's output and a learned vector per pass joining the stream.  The
head is the embedding table, the logits are pressed into (-logit_softcap, logit_softcap).  Keys: `vocab`, `width`,
`logit_softcap`, `embedding.scale`, `norm.eps`, `layers[i].{type, mixer, mlp}`, `loop.{start, stop, times}`;
core/bilurax.cpp lists them all.

Reading, type checks and validation are the host library's (core/bilurax.cpp, BiluraxConfig); this dataclass
carries the result.  Its layer records stay plain dictionaries, as config.json writes them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .. import core
from .base import ModelConfig


@dataclasses.dataclass(frozen=True)
class BiluraxConfig(ModelConfig):
    architecture = "Bilurax"

    vocab: int = 0
    width: int = 0
    logit_softcap: float = 0.0
    embedding: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"scale": 1.0})
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    loop: Optional[Dict[str, Any]] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BiluraxConfig":
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
