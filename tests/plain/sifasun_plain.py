"""Plain, slow statement of the Sifasun decoder: whole sequences, no cache, no batching, one
function per mechanism, CPU float32.  It shares no code with the package under test.

Notation: x is the [tokens, width] residual of one sequence, W matrices are [out, in] and are
applied as x W^T, t and j run over tokens in order, positions count from 0.  `rnd` is where an
engine that stores activations in bfloat16 rounds them (identity for the 32-bit statement).

A layer adds the NORMED output of each sublayer to the residual, and the sublayers read the
residual itself:   x <- x + N1(mixer(x));   x <- x + N2(ff(x)),   N(y) = y / rms(y) * (1 + w).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Mapping, Optional, Sequence

import torch

Tensor = torch.Tensor
Round = Callable[[Tensor], Tensor]


def exact(t: Tensor) -> Tensor:
    return t


def bf16(t: Tensor) -> Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def lin(h: Tensor, w: Tensor) -> Tensor:
    return h.float() @ w.float().t()


# ---------------------------------------------------------------------------------------
# norms


def rms_unit(y: Tensor, eps: float) -> Tensor:
    """y divided by its root mean square over the last axis, eps inside the root."""
    y = y.float()
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def norm_one_plus(y: Tensor, w: Tensor, eps: float) -> Tensor:
    """RMS norm whose stored weight lies around zero."""
    return rms_unit(y, eps) * (1.0 + w.float())


def norm_plain_weight(y: Tensor, w: Tensor, eps: float) -> Tensor:
    return rms_unit(y, eps) * w.float()


# ---------------------------------------------------------------------------------------
# rotation


def rotate_half(v: Tensor, dims: int, base: float, factor: float = 1.0, first_position: int = 0) -> Tensor:
    """v [tokens, heads, dim]: the first `dims` numbers of every head are turned, number i together
    with number i + dims/2, by the angle position * base^(-2i/dims) / factor; the rest pass."""
    T = v.shape[0]
    half = dims // 2
    out = v.clone().float()
    if half == 0:
        return out
    i = torch.arange(half, dtype=torch.float64)
    freq = (torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims) / factor).float()
    pos = torch.arange(first_position, first_position + T, dtype=torch.float32)
    ang = pos[:, None] * freq[None, :]                       # float32 product, as an engine forms it
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half].float(), v[..., half:dims].float()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------
# attention over a sliding window


def window_of(m: Mapping) -> Optional[int]:
    return (m.get("mask") or {}).get("size")


def window_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, window: Optional[int], softcap: Optional[float],
                     sink: bool) -> Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Token t sees j with 0 <= t - j < window (None: all j <= t).
    `softcap` c: score <- c tanh(score / c).  `sink`: one more term exp(0) in the softmax's denominator
    that carries no value."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1])
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, g].float() @ q[t, h].float()) * scale
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            m = s.max()
            if sink:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(-m) if sink else 0.0)
            out[t, h] = (e / den) @ v[lo:t + 1, g].float()
    return out


def attention_mixer(x: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Keys double as values (as projected); rotation on part of each head with stretched positions; unit
    RMS per head after the rotation; capped scores; softmax with a sink."""
    T = x.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    h = rnd(x)
    q = lin(h, p["q"]).view(T, H, D)
    k = lin(h, p["k"]).view(T, G, D)
    v = rnd(k)
    rot = m["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rms_unit(rotate_half(q, rot["dims"], rot["base"], factor), eps)
    k = rms_unit(rotate_half(k, rot["dims"], rot["base"], factor), eps)
    o = window_attention(rnd(q), rnd(k), v, float(m["scale"]), window_of(m), m.get("softcap"), sink=True)
    return lin(rnd(o.reshape(T, -1)), p["o"])


def left_mixer(x: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Keys double as values; one RMS norm over the whole query projection (and one over the whole key
    projection) with plain weights, before the rotation; ordinary softmax."""
    T = x.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    h = rnd(x)
    q = lin(h, p["left.q"])
    k = lin(h, p["left.k"])
    v = rnd(k).view(T, G, D)
    q = norm_plain_weight(q, p["left.q.norm"], eps).view(T, H, D)
    k = norm_plain_weight(k, p["left.k.norm"], eps).view(T, G, D)
    rot = m["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_half(q, rot["dims"], rot["base"], factor)
    k = rotate_half(k, rot["dims"], rot["base"], factor)
    o = window_attention(rnd(q), rnd(k), v, float(m["scale"]), window_of(m), m.get("softcap"), sink=False)
    return lin(rnd(o.reshape(T, -1)), p["left.o"])


# ---------------------------------------------------------------------------------------
# the gated linear recurrence


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(u: Tensor, taps: Tensor, bias: Tensor) -> Tensor:
    """u [T, C], taps [C, K]: out[t] = bias + sum_j taps[:, K-1-j] u[t-j], zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C), u.float()], dim=0)
    out = bias.float().expand(T, C).clone()
    for j in range(K):
        out = out + pad[j:j + T] * taps[:, j].float()
    return out


def block_gate(u: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """sigmoid of a block-diagonal map: u [T, C] in `blocks` equal parts, w [blocks, n, n] ([out, in]), b [blocks, n]."""
    T, C = u.shape
    nb = w.shape[0]
    parts = u.float().view(T, nb, C // nb)
    z = torch.einsum("tbi,boi->tbo", parts, w.float()) + b.float()
    return torch.sigmoid(z).reshape(T, C)


def gated_recurrence(u: Tensor, r: Tensor, i: Tensor, lam: Tensor) -> Tensor:
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, a_t = exp(-8 r_t softplus(lam)), per channel."""
    T, C = u.shape
    log_a = -8.0 * r * torch.nn.functional.softplus(lam.float())
    a = torch.exp(log_a)
    mult = torch.sqrt(1.0 - a * a)
    S = torch.zeros(C)
    out = torch.zeros(T, C)
    for t in range(T):
        S = a[t] * S + mult[t] * i[t] * u[t]
        out[t] = S
    return out


def right_mixer(x: Tensor, p: Mapping[str, Tensor], m: Mapping, rnd: Round = exact) -> Tensor:
    h = rnd(x)
    y = rnd(gelu_tanh(lin(h, p["right.y"]) + p["right.y.b"].float()))
    u = causal_conv(rnd(lin(h, p["right.x"]) + p["right.x.b"].float()), p["right.conv"], p["right.conv.b"])
    r = block_gate(u, p["right.ra"], p["right.ra.b"])
    i = block_gate(u, p["right.ri"], p["right.ri.b"])
    S = gated_recurrence(u, r, i, p["right.lam"])
    return lin(rnd(S * y), p["right.o"])


def parallel_mixer(x: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    return (float(m["left_scale"]) * left_mixer(x, p, m["left"], eps, rnd)
            + float(m["right_scale"]) * right_mixer(x, p, m["right"], rnd))


# ---------------------------------------------------------------------------------------
# feed-forward, the model


def dense_ff(x: Tensor, p: Mapping[str, Tensor], rnd: Round = exact) -> Tensor:
    h = rnd(x)
    g = lin(h, p["gate"])
    return lin(rnd(g * torch.sigmoid(g) * lin(h, p["up"])), p["down"])


def sub(weights: Mapping[str, Tensor], prefix: str) -> Dict[str, Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: Mapping, weights: Mapping[str, Tensor], tokens: Sequence[int], rnd: Round = exact,
            residuals: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [tokens, vocab] of one sequence.  `residuals`, if a list, receives the residual after every layer."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"].float()[torch.as_tensor(list(tokens), dtype=torch.long)]
    for li, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", li)
        pre = f"l{src}."
        mix = sub(weights, pre + "mix.")
        if layer["type"] == "parallel":
            y = parallel_mixer(x, mix, layer["mixer"], eps, rnd)
        elif layer["type"] == "attention":
            y = attention_mixer(x, mix, layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, weights[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_one_plus(dense_ff(x, sub(weights, pre + "mlp."), rnd), weights[pre + "norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    hn = norm_one_plus(x, weights["final.norm"], eps)
    return lin(rnd(hn), weights["embed"]) * float(config["logit_scale"])
