"""RMSNorm: out = x * w / sqrt(mean(x^2) + eps), eps inside the root, the scale multiplies
plainly (src/ops/rmsnorm.rs:38-48).  Statistics in fp32 on the fp32 residual stream.  With the spec's
`offset` c the stored weight lies around zero and the scale is c + w (formed once, in fp32)."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import LazyInput, Norm, NormRequest, Runtime, register_part


class ScaledRows(LazyInput):
    """An RMSNorm of the fp32 rows `rows` whose first half is done: `scaled` = bf16(rows * weight) and
    `sumsq` [rows, parts] (partial sums of squares of each row) were written by the kernel that wrote
    `rows`; each row's factor 1 / sqrt(mean + eps) is still to be applied, by the projection that
    reads `scaled` (to its outputs: the product is linear in its input)."""

    def __init__(self, norm: "RMSNorm", rows, scaled, sumsq, parts: int, ctx):
        self.norm, self.rows, self.scaled, self.sumsq, self.parts, self.ctx = norm, rows, scaled, sumsq, parts, ctx

    def row_scale(self) -> B.RowScale:
        return B.RowScale(sumsq=self.sumsq.data_ptr(), parts=self.parts, hidden=self.norm.hidden_size, eps=self.norm.eps)

    def materialize(self, n_rows: int):
        out = self.norm.rt.workspace.take("block.normed", self.rows.shape, self.norm.rt.dtype)
        self.norm.forward(self.rows, out, self.ctx, rows=n_rows)
        return out


def honour(request: NormRequest, rows, ctx, name: str, max_parts: int):
    """For a kernel about to write the fp32 `rows`: the buffers of the norm's first half and the
    kernel argument that names them.  `finish(ahead)` (after the launch) makes the `ScaledRows`."""
    ws = request.norm.rt.workspace
    scaled = ws.take(name + ".ahead_scaled", rows.shape, torch.bfloat16)
    sumsq = ws.take(name + ".ahead_sumsq", (rows.shape[0], max_parts), torch.float32)
    ahead = B.norm_ahead(request.weight, scaled, sumsq)

    def finish():
        return ScaledRows(request.norm, rows, scaled, sumsq, int(ahead.parts), ctx) if ahead.parts > 0 else None
    return ahead, finish


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, hidden_size: int, rt: Runtime):
        self.eps = float(spec["eps"])
        self.offset = float(spec.get("offset", 0.0))
        self.hidden_size = hidden_size
        self.rt = rt
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden_size,), "normal" if self.offset else "ones_plus_normal")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = tensors["weight"]
        self.weight = (w.to(torch.float32) + self.offset).contiguous() if self.offset else w.contiguous()
        self._weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.to(torch.float32)

    def add_normed(self, y, x, cast, ctx, rows: int) -> None:
        """x[:rows] += norm(y[:rows]) for a layer that norms a sublayer's output (fp32 both); clears y's rows
        for the sublayer to come and writes the new rows into `cast` (the run's dtype, optional)."""
        B.add_normed(x, y, self._weight_f32, cast, rows, self.eps, ctx.stream)

    def forward(self, x, out, ctx, rows_idx=None, rows=None) -> None:
        B.rmsnorm(x, self.weight, out, self.eps, ctx.stream, rows_idx=rows_idx, rows=rows)

    def request_ahead(self):
        return NormRequest(self, self.weight, self.eps)


class LayerNorm(Norm):
    """out = (x - mean) / sqrt(var + eps) * weight + b, var = mean((x - mean)^2), statistics in fp32.
    Tensors: "weight" and the bias "b" (found at the weight's name + ".b").

    `forward_streams` is the same norm for a residual kept as S streams per token (hyper-connections):
    one kernel updates the streams with the output `y` of the sublayer before (x'_t = sum_s mix[s, t] x_s
    + outc[t] y), clears y for the sublayer to come, combines u = sum_s in_coef[s] x'_s and norms u."""
    graph_safe = True

    def __init__(self, spec, hidden_size: int, rt: Runtime):
        self.eps = float(spec["eps"])
        self.hidden_size = hidden_size
        self.rt = rt
        self.weight = None
        self.bias = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden_size,), "ones_plus_normal"), "b": TensorSpec((self.hidden_size,))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["b"].to(torch.float32).contiguous()

    def forward(self, x, out, ctx, rows_idx=None, rows=None) -> None:
        n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else x.shape[0])
        B.streams_norm(x, 1, self.hidden_size, n, ctx.stream, w=self.weight, b=self.bias, eps=self.eps, out=out,
                       rows_idx=rows_idx)

    def forward_streams(self, xs, n_streams: int, out, ctx, rows: int, rows_idx=None, in_coef=None, update=None,
                        clear=None) -> None:
        """`update` = (y, mix [S, S] indexed [from, to], outc [S]): apply and store the streams' update first;
        `clear`: a [tokens, hidden] fp32 buffer whose rows are zeroed (the next sublayer adds into it)."""
        y, mix, outc = update if update is not None else (clear, None, None)
        B.streams_norm(xs, n_streams, self.hidden_size, rows, ctx.stream, y=y, mix=mix, outc=outc,
                       update=update is not None, write_back=update is not None, zero_y=clear is not None,
                       in_coef=in_coef, w=self.weight, b=self.bias, eps=self.eps, out=out, rows_idx=rows_idx)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
