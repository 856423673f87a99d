"""Latent attention without positions, with a softmax sink.

Queries go through a latent: c_q = RMSnorm(W_dq h) (plain weight), q = W_uq c_q (heads x dim).  Keys and
values come from one shared latent per token, c = RMSnorm(W_dkv h) with kv_rank numbers, the only thing
the cache keeps: k = W_uk c, v = W_uv c per head (dim and vdim may differ).  Causal softmax of
(q . k) * scale with a sink: each head has a learned logit sink_h that only enlarges the denominator by
exp(sink_h), taken unscaled, and adds nothing to the weighted sum; then W_o on the concatenated heads.

A prompt expands k and v for its own tokens and attends over them.  A one-token step attends over the
cached latents in the absorbed form: the query is taken into the latent's coordinates (W_uk^T q), the
scores and the weighted sum are formed on the latents themselves, and W_uv is applied once to the sum,
so nothing is expanded per cached position.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import KVRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, register_part
from .linear import Linear


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.H, self.D, self.V = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.q_rank, self.kv_rank = int(spec["q_rank"]), int(spec["kv_rank"])
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, hd, hv = self.hidden_size, self.H * self.D, self.H * self.V
        return {"dq": TensorSpec((self.q_rank, h)), "dq.norm": TensorSpec((self.q_rank,), "ones_plus_normal"),
                "uq": TensorSpec((hd, self.q_rank)),
                "dkv": TensorSpec((self.kv_rank, h)), "dkv.norm": TensorSpec((self.kv_rank,), "ones_plus_normal"),
                "uk": TensorSpec((hd, self.kv_rank)), "uv": TensorSpec((hv, self.kv_rank)),
                "sink": TensorSpec((self.H,)), "o": TensorSpec((h, hv))}

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        self.down = Linear(torch.cat([t["dq"].to(dt), t["dkv"].to(dt)], dim=0), self.rt)
        self.uq = Linear(t["uq"], self.rt)
        self.ukv = Linear(torch.cat([t["uk"].to(dt), t["uv"].to(dt)], dim=0), self.rt)
        self.w_uk = self.ukv.weight[:self.H * self.D]           # views, for the absorbed form
        self.w_uv = self.ukv.weight[self.H * self.D:]
        self.q_norm, self.kv_norm = t["dq.norm"].to(torch.float32).contiguous(), t["dkv.norm"].to(torch.float32).contiguous()
        self.sink = t["sink"].to(torch.float32).contiguous()
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> KVRequest:
        return KVRequest(kv_heads=1, head_dim=self.kv_rank, window=None, values=False)

    def weight_bytes(self) -> int:
        return self.down.nbytes() + self.uq.nbytes() + self.ukv.nbytes() + self.o.nbytes()

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, H, D, V = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.D, self.V
        kv = cache_view.struct
        lat = ws.take("latent.down", (T, self.q_rank + self.kv_rank), torch.float32)
        self.down.apply(xn, lat, T, ctx.stream)
        cq = ws.take("latent.cq", (T, self.q_rank), rt.dtype)
        c = ws.take("latent.c", (T, self.kv_rank), rt.dtype)
        B.latent_norm_store(lat, self.q_rank, self.kv_rank, self.q_norm, self.kv_norm, self.eps, cq, c, ctx.batch, kv,
                            writes_cache, rt.err, ctx.stream)
        out = ws.take("latent.out", (T, H * V), rt.dtype)
        if ctx.kind == "prompt" and writes_cache:
            qkv = ws.take("latent.qkv", (T, 2 * H * D + H * V), rt.dtype)
            self.uq.apply(cq, qkv[:, :H * D], T, ctx.stream)
            self.ukv.apply(c, qkv[:, H * D:], T, ctx.stream)
            # keys and values of one size: the tensor-core prompt attention (tcgen05 at 64 and 128), with
            # every head its own key/value head and the sink in the denominator
            if not (rt.fast and qkv.dtype == torch.bfloat16 and D == V and
                    B.attention_prefill(qkv, out, ctx.batch, H, H, D, 0, self.scale, ctx.max_q_len, ctx.stream,
                                        err=rt.err, sink=self.sink)):
                B.latent_attention_prompt(qkv, out, ctx.batch, H, D, V, self.scale, self.sink, ctx.stream)
        else:
            q = ws.take("latent.q", (T, H * D), rt.dtype)
            self.uq.apply(cq, q, T, ctx.stream)
            done = False
            if rt.fast and q.dtype == torch.bfloat16 and ctx.kind == "decode":
                hpad, splits = B.latent_decode_tc_plan(ctx.n_seqs, H, cache_view.group.table_width)
                rank = self.kv_rank
                qa = ws.take("latent.qa", (T, hpad, rank), torch.bfloat16)
                part_m = ws.take("latent.part_m", (T, splits, hpad), torch.float32)
                part_l = ws.take("latent.part_l", (T, splits, hpad), torch.float32)
                part_acc = ws.take("latent.part_acc", (T, splits, hpad, rank), torch.float32)
                done = B.latent_attention_decode_tc(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale,
                                                    self.sink, hpad, splits, qa, part_m, part_l, part_acc, rt.err, ctx.stream)
            if not done:
                B.latent_attention_decode(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale, self.sink,
                                          rt.err, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


register_part("mixer", "latent_attention", LatentAttention)
