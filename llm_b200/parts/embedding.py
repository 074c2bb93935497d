"""Token embedding in, logits out.

Embedding: a row copy without scaling (kernel/embedding/TokenEmbedding.h:12-17),
written straight into the float32 residual stream.  Head: logits = rows W^T in
float32 at the rows that were asked for; untied unless the spec ties it to the
embedding table (model/modules/LMHead.h:5-13 is always untied and runs every row).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, ResidualStream, register_part
from .linear import linear


class TokenEmbedding(Part):
    role = "embedding"

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str = "weight", copies: int = 1, scale: float = 1.0,
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.scale = float(scale)             # every row is multiplied by it (float32) on its way into the stream
        if self.scale != 1.0 and int(copies) > 1:
            raise ValueError("token embedding: a scale goes with one copy of the stream")
        self.copies = int(copies)             # a stream kept as several copies: each starts as the embedding
        self.weight_name = weight_name        # "": the table is the tensor named like the part
        self.table = None

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        self.table = tensors[self.name(self.weight_name)].contiguous()

    def forward(self, ctx, stream: ResidualStream) -> None:
        if self.copies > 1:
            ops.hc_embedding(stream.resid, self.table, ctx.token_ids, ctx.n_tokens, self.copies, ctx.status)
        else:
            ops.embedding(stream.resid, self.table, ctx.token_ids, ctx.n_tokens, ctx.status, self.scale)
        stream.pending = stream.pending_post = None


class LMHead(Part):
    role = "head"

    def __init__(self, hidden_size: int, vocab_size: int, tied_to=None, weight_name: str = "weight", softcap=None,
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.hidden_size, self.vocab_size, self.tied_to = hidden_size, vocab_size, tied_to
        self.softcap = float(softcap) if softcap else None      # logits <- cap * tanh(logits / cap)
        self.weight_name = weight_name        # "": the matrix is the tensor named like the part
        self.weight = None

    def parameters(self):
        if self.tied_to:
            return {}
        return {self.name(self.weight_name): ParamInfo((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to else self.name(self.weight_name)].contiguous()

    def forward(self, rows: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        return linear(rows, self.weight, out, n_rows)

    def logits(self, stream: ResidualStream, ctx, final_norm, buffers) -> torch.Tensor:
        """Everything after the last layer: the wanted rows of the stream (with its pending term)
        are gathered, normalised by final_norm (None: the model has none) and projected.  buffers:
        (float32 rows, rows in the compute dtype, float32 logits), each with room for
        ctx.n_logit_rows rows, at addresses that stay fixed between steps."""
        rows, normed, out = buffers
        R = ctx.n_logit_rows
        if stream.pending is not None and stream.pending_post is not None:
            stream.fold(ctx)          # a term that is still to be normed cannot be gathered as it is
        copies = stream.resid.shape[1] // self.hidden_size
        if copies > 1:                # a stream kept as several copies: the model's output is their sum
            stream.fold(ctx)
            ops.hc_gather_sum(rows, stream.resid, ctx.logit_rows, R, copies)
        else:
            ops.gather_rows(rows, stream.resid, stream.pending, ctx.logit_rows, R)
        if final_norm is not None:
            final_norm.forward_rows(rows, R, normed)
        else:
            ops.cast_rows(normed, rows, R)
        res = linear(normed, self.weight, out, R)
        if self.softcap:
            ops.softcap(out, R, self.softcap)
        return res


class EmbeddingReinjection(Part):
    """x <- W [x ; e] + b_pass: the stream is mixed anew with the embedding e of the same tokens, as a stack of
    layers that runs several times with the same weights does at the start of each pass.  W is
    [hidden, 2 hidden] with the stream's half first; `steps` is [passes, hidden] and row `pass_index` of it
    is added.  The product takes its inputs in the compute dtype and accumulates in float32; its result
    replaces the float32 residual."""

    role = "stream"

    def __init__(self, hidden_size: int, vocab_size: int, passes: int, pass_index: int, table_name: str, in_name: str = "in",
                 step_name: str = "step", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if not (0 <= pass_index < passes):
            raise ValueError(f"embedding re-injection: pass {pass_index} of {passes}")
        self.hidden_size, self.vocab_size, self.passes, self.pass_index = hidden_size, vocab_size, passes, pass_index
        self.table_name, self.in_name, self.step_name = table_name, in_name, step_name
        self.table = self.w = self.step = None

    def parameters(self):
        return {self.table_name: ParamInfo((self.vocab_size, self.hidden_size)),
                self.name(self.in_name): ParamInfo((self.hidden_size, 2 * self.hidden_size)),
                self.name(self.step_name): ParamInfo((self.passes, self.hidden_size), kind="gain", init="normal")}

    def bind(self, tensors):
        self.table = tensors[self.table_name].contiguous()
        self.w = tensors[self.name(self.in_name)].contiguous()
        self.step = tensors[self.name(self.step_name)][self.pass_index].contiguous()

    def forward(self, stream: ResidualStream, ctx) -> None:
        T = stream.rows
        stream.fold(ctx)
        both = ctx.workspace.get("stream_and_embedding", T, 2 * self.hidden_size, self.dtype)
        ops.concat_embedding(both, stream.resid, self.table, ctx.token_ids, T)
        linear(both, self.w, stream.resid, T, bias=self.step)


register_part("stream", "embedding_reinjection", EmbeddingReinjection)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
