"""A recurrent block with two branches and a real-gated linear recurrent unit (the recurrent block of
Griffin: De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language
Models").  With h the mixer's input and C = `width` channels:

    g = gelu_tanh(W_y h + b_y)
    u = conv(W_x h + b_x)             a causal convolution per channel over `conv` taps (the last tap is the
                                      current token's), with a bias, zeros before the sequence's start
    r = sigmoid(R_a u + b_a),  i = sigmoid(R_i u + b_i)       block-diagonal: `blocks` square matrices
    log a = -c r softplus(lam),  S_t = a S_(t-1) + sqrt(1 - a^2) i u      (c = `decay_constant`, default 8)
    result = W_o (S g) * out_scale

State per sequence (fp32, zero at the start, carried from step to step): S and the convolution's last
conv - 1 inputs.  Tensors: y, y.b, x, x.b, conv [C, taps], conv.b, ra / ri [blocks, C/blocks, C/blocks],
ra.b / ri.b [blocks, C/blocks], lam [C], o [hidden, C].

One product makes [W_y h | W_x h] in fp32; the convolution, the gates and the scan are the kernels of
`csrc/rglru.cu` (all fp32); W_o is added into the residual.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, register_part
from .linear import Linear


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class RecurrentGatedUnit(Mixer):
    graph_safe = True
    takes_out_scale = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.C = int(spec["width"])
        self.blocks = int(spec["blocks"])
        self.taps = int(spec["conv"])
        self.decay_constant = float(spec.get("decay_constant", 8.0))
        self.out_scale = float(spec.get("out_scale", 1.0))
        if self.C % self.blocks:
            raise ValueError(f"width {self.C} is not a multiple of blocks {self.blocks}")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv must be between 1 and 16 taps, got {self.taps}")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, C, nb = self.hidden_size, self.C, self.blocks
        bw = C // nb
        return {"y": TensorSpec((C, h)), "y.b": TensorSpec((C,)), "x": TensorSpec((C, h)), "x.b": TensorSpec((C,)),
                "conv": TensorSpec((C, self.taps)), "conv.b": TensorSpec((C,)),
                "ra": TensorSpec((nb, bw, bw)), "ra.b": TensorSpec((nb, bw)),
                "ri": TensorSpec((nb, bw, bw)), "ri.b": TensorSpec((nb, bw)),
                "lam": TensorSpec((C,)), "o": TensorSpec((h, C))}

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        self.proj = Linear(torch.cat([t["y"].to(dt), t["x"].to(dt)], dim=0), self.rt)
        self.by, self.bx = _f32(t["y.b"]), _f32(t["x.b"])
        self.conv_w, self.conv_b = _f32(t["conv"]), _f32(t["conv.b"])
        self.ra, self.ri = t["ra"].to(dt).contiguous(), t["ri"].to(dt).contiguous()
        self.ra_b, self.ri_b = _f32(t["ra.b"]).view(-1), _f32(t["ri.b"]).view(-1)
        self.lam = _f32(t["lam"])
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> StateRequest:
        return StateRequest((self.C * self.taps,), torch.float32)

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + 2 * self.ra.numel() * self.ra.element_size()

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, C = self.rt, self.rt.workspace, ctx.n_tokens, self.C
        state = cache_view.state
        proj = ws.take("rglru.proj", (T, 2 * C), torch.float32)
        self.proj.apply(xn, proj, T, ctx.stream)
        u = ws.take("rglru.u", (T, C), torch.float32)
        B.rglru_conv(proj, self.bx, self.conv_w, self.conv_b, state, u, C, self.taps, ctx.batch, ctx.stream)
        a = ws.take("rglru.a", (T, C), torch.float32)
        bv = ws.take("rglru.b", (T, C), torch.float32)
        B.rglru_gates(u, self.ra, self.ra_b, self.ri, self.ri_b, self.lam, self.decay_constant, a, bv, T, C, self.blocks,
                      ctx.stream)
        out = ws.take("rglru.out", (T, C), rt.dtype)
        scratch = None
        if ctx.kind == "prompt" and ctx.max_q_len > 128:       # long prompts: the scan in chunks
            scratch = ws.take("rglru.chunks", (B.rglru_scan_scratch_floats(ctx.n_seqs, ctx.max_q_len, C),), torch.float32)
        B.rglru_scan(a, bv, proj, self.by, self.bx, state, out, self.out_scale, C, self.taps, ctx.batch, ctx.stream,
                     max_q_len=ctx.max_q_len, scratch=scratch)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


register_part("mixer", "rglru", RecurrentGatedUnit)
