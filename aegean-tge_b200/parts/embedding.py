"""Token embedding and output head.

Embedding is a row copy with no scaling (src/models/qwen2.cpp:1143-1152,
:2050); the head is a plain product of the final-normed rows with the output
matrix, which is the embedding table itself when the model ties them
(src/models/qwen2.cpp:412-420, :2121-2122).  Logits are float32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import EMBEDDINGS, HEADS, NORMS, ParamSpec, Part, build_part


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: ``vocab_size``, ``hidden_size``; optional ``norm`` (a norm's PartSpec: the looked-up rows are
    normalised before they become the stream; the norm needs ``forward_stream``), ``scale`` (a factor on the looked-up
    rows, default 1; a head that shares the table reads it unscaled).  weights: ``weight`` and, with a
    norm, its parameters as ``norm.<name>``."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight: Optional[torch.Tensor] = None
        norm = spec.params.get("norm")
        self.norm = build_part(NORMS, norm, env) if norm is not None else None
        if self.norm is not None and not hasattr(self.norm, "forward_stream"):
            raise ValueError(f"token_embedding: norm '{norm.kind}' cannot normalise the stream in place")

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"weight": ParamSpec((self.vocab, self.hidden))}
        if self.norm is not None:
            specs.update({f"norm.{name}": param for name, param in self.norm.param_specs().items()})
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]
        if self.norm is not None:
            self.norm.load({name[len("norm."):]: t for name, t in tensors.items() if name.startswith("norm.")})

    def param_bytes(self) -> int:
        return 0        # a step reads the rows of its tokens, not the table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = self.ops.embedding(self.weight, token_ids, scale=self.scale)
        return x if self.norm is None else self.norm.forward_stream(x)


@HEADS.register("linear_head")
class LinearHead(Part):
    """params: ``vocab_size``, ``hidden_size``; optional ``logit_scale`` (multiplies the logits, in the product's
    epilogue) and ``soft_cap`` (then logits <- cap * tanh(logits / cap), float32).  weights: ``weight`` [vocab, hidden]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.logit_scale = float(spec.params.get("logit_scale", 1.0))
        cap = spec.params.get("soft_cap")
        self.cap = None if cap is None else float(cap)
        if self.cap is not None and not self.cap > 0.0:
            raise ValueError("linear_head: soft_cap must be positive")
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * self.vocab * self.hidden

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.ops.linear(h, self.weight, None, self.ops.GEMM_STORE_F32, alpha=self.logit_scale)
        return logits if self.cap is None else self.ops.soft_cap(logits, self.cap)
