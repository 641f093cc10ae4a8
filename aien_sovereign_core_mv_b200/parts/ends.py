"""The two ends of the model: the token embedding and the output head."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import make_part, register_embedding, register_head, register_pass_input
from .base import Embedding, Head, Part, StepContext
from .linear import linear


@register_embedding("table")
class TableEmbedding(Embedding):
    """x[t] = weight[token_ids[t]], widened to float32 (crates/aien-inference-abi/src/
    transformer_backend.rs:1179-1181, src/weights.rs:140-146; ids are checked against the
    vocabulary before a step is accepted instead of being reduced modulo it).

    ``scale``: the row is multiplied by this constant.  ``side_width`` > 0: the part also owns a second table
    ``side`` [vocab, side_width] that it does not read itself; layers with a per-token side input take their columns
    of it (``side_table``).  ``sinusoid_base`` b > 0: the sinusoidal vector of the token's position is added, entry
    2i = sin(p * b^(-2i/hidden)), entry 2i+1 = cos of the same angle (the angle in float64, as the rotary tables)."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, side_width: int = 0, sinusoid_base: float = 0.0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.side_width = float(scale), int(side_width)
        self.sinusoid_base = float(sinusoid_base or 0.0)
        self.weight: Optional[torch.Tensor] = None
        self.side: Optional[torch.Tensor] = None
        self.inv_freq: Optional[torch.Tensor] = None

    def param_shapes(self):
        shapes = {"weight": ((self.vocab_size, self.hidden_size), "embedding")}
        if self.side_width > 0:
            shapes["side"] = ((self.vocab_size, self.side_width), "embedding")
        return shapes

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()
        if self.side_width > 0:
            self.side = tensors["side"].contiguous()
        if self.sinusoid_base > 0.0:
            H = self.hidden_size
            f = [self.sinusoid_base ** (-2.0 * i / H) for i in range((H + 1) // 2)]
            self.inv_freq = torch.tensor(f, dtype=torch.float64, device=self.weight.device)

    def tied_weight(self):
        return self.weight

    def side_table(self) -> Optional[torch.Tensor]:
        return self.side

    def _gather(self, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        if self.scale != 1.0:
            K.embed_gather_scaled(self.weight, token_ids, x, self.scale)
        else:
            K.embed_gather(self.weight, token_ids, x)

    def forward(self, ctx: StepContext, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        if self.inv_freq is not None:
            K.embed_gather_sinusoid(self.weight, token_ids, ctx.positions, self.inv_freq, x, self.scale)
        else:
            self._gather(token_ids, x)


@register_embedding("table_normed")
class NormedTableEmbedding(TableEmbedding):
    """x[t] = norm(weight[token_ids[t]]): a table whose rows pass a norm before they become the
    residual stream.  ``norm`` names a registered norm part ({"kind": ..., further parameters});
    its tensors are this part's ``norm.<local name>``.  A head tied to this embedding multiplies
    by the table itself."""

    def __init__(self, vocab_size: int, hidden_size: int, norm: dict, scale: float = 1.0, side_width: int = 0):
        super().__init__(vocab_size, hidden_size, scale, side_width, 0.0)
        params = {k: v for k, v in dict(norm).items() if k != "kind"}
        self.norm = make_part("norm", norm["kind"], size=self.hidden_size, **params)
        if not hasattr(self.norm, "norm_stream"):
            raise ValueError(f"norm kind {norm['kind']!r} cannot norm the stream in place")

    def param_shapes(self):
        shapes = dict(super().param_shapes())
        for local, spec in self.norm.param_shapes().items():
            shapes[f"norm.{local}"] = spec
        return shapes

    def bind(self, tensors):
        super().bind(tensors)
        self.norm.bind({k[len("norm."):]: v for k, v in tensors.items() if k.startswith("norm.")})

    def forward(self, ctx: StepContext, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        self._gather(token_ids, x)
        self.norm.norm_stream(ctx, x)


@register_head("linear")
class LinearHead(Head):
    """logits = rows . W^T with W = ``weight`` [vocab, hidden], or the embedding's table when
    tied: the same buffer, no copy (crates/aien-inference-abi/src/weights.rs:131-136,
    src/transformer_backend.rs:1370-1386).  ``softcap`` c > 0: logits = c * tanh(logits / c), in float32."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False, softcap: float = 0.0):
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.softcap = float(softcap or 0.0)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {} if self.tied else {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: Embedding) -> None:
        w = embedding.tied_weight()
        if w is None or tuple(w.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("the head is tied to an embedding that offers no [vocab, hidden] matrix")
        self.weight = w

    def forward(self, ctx: StepContext, rows: torch.Tensor, logits: torch.Tensor) -> None:
        linear(ctx, rows, self.weight, out=logits)
        if self.softcap > 0.0:
            K.softcap(logits, self.softcap)


@register_pass_input("step_vector")
class StepVectorInput(Part):
    """What a stretch of layers that runs ``times`` times in a row adds to the stream before pass t = 0, 1, ...: the
    embedding's output once more (``add_embedding``; every pass but the first), then the row t of ``steps`` [times,
    hidden] for every token.  The sums are float32."""

    def __init__(self, hidden_size: int, times: int, add_embedding: bool = True):
        self.hidden_size, self.times, self.add_embedding = int(hidden_size), int(times), bool(add_embedding)
        if self.times <= 0:
            raise ValueError(f"times {times!r} must be positive")
        self.steps: Optional[torch.Tensor] = None

    @property
    def wants_embedding(self) -> bool:
        """Whether the decoder keeps the embedding's output for this part."""
        return self.add_embedding and self.times > 1

    def param_shapes(self):
        return {"steps": ((self.times, self.hidden_size), "small")}

    def bind(self, tensors):
        self.steps = tensors["steps"].contiguous()

    def forward(self, ctx: StepContext, x: torch.Tensor, embedded: Optional[torch.Tensor], t: int) -> None:
        if not (0 <= t < self.times):
            raise ValueError(f"pass {t} of {self.times}")
        K.pass_input(x, embedded if (self.add_embedding and t > 0) else None, self.steps[t])
