"""Plain, slow statement of the Vefulix decoder: whole sequences, no cache, no batching, one
function per mechanism, CPU float32.  It shares no code with the package under test.

Notation: h is a [tokens, width] matrix of one sequence, W matrices are [out, in] and are
applied as h W^T, t runs over tokens in order.  `rnd` is where an engine that stores its
activations in bfloat16 rounds them (identity for the 32-bit statement).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Mapping, Optional, Sequence

import torch
import torch.nn.functional as F

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


def layer_norm(x: Tensor, w: Tensor, b: Tensor, eps: float) -> Tensor:
    x = x.float()
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.float() + b.float()


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x divided by its root mean square over the last axis."""
    x = x.float()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------------------------------
# mixers (one sequence each)


def mlstm_mixer(h: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Matrix memory with exponential input gate and a running maximum that starts at 0."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = rnd(lin(h, p["q"])).view(T, H, D) * D ** -0.5
    k = rnd(lin(h, p["k"])).view(T, H, D)
    v = rnd(lin(h, p["v"])).view(T, H, V)
    gi = cap * torch.tanh((lin(h, p["i"]) + p["i.b"].float()) / cap)                     # [T, H]
    gf = F.logsigmoid(cap * torch.tanh((lin(h, p["f"]) + p["f.b"].float()) / cap))
    out = torch.zeros(T, H, V)
    for hd in range(H):
        S = torch.zeros(D, V)
        n = torch.zeros(D)
        mx = torch.zeros(())
        for t in range(T):
            new = torch.maximum(gf[t, hd] + mx, gi[t, hd])
            a, b = torch.exp(gf[t, hd] + mx - new), torch.exp(gi[t, hd] - new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = new
            den = torch.maximum((n @ q[t, hd]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hd] = (S.t() @ q[t, hd]) / den
    o = rms_unit(out, eps).reshape(T, H * V) * p["norm"].float()
    o = o * torch.sigmoid(rnd(lin(h, p["g"])))
    return lin(rnd(o), p["o"])


def causal_conv_silu(x: Tensor, taps: Tensor) -> Tensor:
    """y[t, c] = silu(sum_j taps[c, K-1-j] x[t-j, c]), zeros before the first token."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros(T, C)
    for j in range(K):
        shifted = torch.zeros(T, C)
        shifted[j:] = x[:T - j] if j else x
        y = y + shifted * taps[:, K - 1 - j].float()
    return F.silu(y)


def delta_mixer(h: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Gated delta rule with short convolutions on q, k, v."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(rnd(lin(h, p["q"])), p["q.conv"]).view(T, G, D)
    k = causal_conv_silu(rnd(lin(h, p["k"])), p["k.conv"]).view(T, G, D)
    v = causal_conv_silu(rnd(lin(h, p["v"])), p["v.conv"]).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, p["b"]))                                                   # [T, H]
    decay = torch.exp(-torch.exp(p["A_log"].float()) * F.softplus(lin(h, p["a"]) + p["dt_bias"].float()))
    out = torch.zeros(T, H, V)
    rep = H // G
    for hd in range(H):
        g = hd // rep
        S = torch.zeros(D, V)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.t() @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.t() @ q[t, g]
    o = rms_unit(out, eps) * p["norm"].float()                                             # weight over vdim, shared by heads
    o = o.reshape(T, H * V) * F.silu(rnd(lin(h, p["g"])))
    return lin(rnd(o), p["o"])


def latent_attention_mixer(h: Tensor, p: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Attention whose keys and values are expanded from one low-rank row per token; the softmax's
    denominator holds one more term exp(sink) per head."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    cq = rnd(rms_unit(lin(h, p["dq"]), eps) * p["dq.norm"].float())
    q = rnd(lin(cq, p["uq"])).view(T, H, D)
    c = rnd(rms_unit(lin(h, p["dkv"]), eps) * p["dkv.norm"].float())
    k = rnd(lin(c, p["uk"])).view(T, H, D)
    v = rnd(lin(c, p["uv"])).view(T, H, V)
    out = torch.zeros(T, H, V)
    mask = torch.ones(T, T).tril().bool()
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd].t()) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        sink = p["sink"].float()[hd]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        w = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
        out[:, hd] = w @ v[:, hd]
    return lin(rnd(out.reshape(T, H * V)), p["o"])


MIXERS = {"mlstm": mlstm_mixer, "delta": delta_mixer, "latent_attention": latent_attention_mixer}


# ---------------------------------------------------------------------------------------
# feed-forward


def gated_ff(h: Tensor, gate: Tensor, up: Tensor, down: Tensor, rnd: Round = exact) -> Tensor:
    return lin(rnd(F.silu(lin(h, gate)) * lin(h, up)), down)


def route(h: Tensor, w: Tensor, b: Tensor, top: int):
    """Chosen experts [T, top] and their weights: softmax over the chosen logits only."""
    z = lin(h, w) + b.float()
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h: Tensor, p: Mapping[str, Tensor], mlp: Mapping, rnd: Round = exact) -> Tensor:
    T = h.shape[0]
    idx, wt = route(h, p["router"], p["router.b"], int(mlp["router"]["top"]))
    out = torch.zeros(T, p["e0.down"].shape[0])
    for t in range(T):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * gated_ff(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"], rnd)[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, p["shared.gate"], p["shared.up"], p["shared.down"], rnd)
    return out


# ---------------------------------------------------------------------------------------
# the model


def sub(tensors: Mapping[str, Tensor], prefix: str) -> Dict[str, Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: Mapping, tensors: Mapping[str, Tensor], tokens: Sequence[int], rnd: Round = exact,
            layer_sums: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [tokens, vocab] of one sequence.  `layer_sums` receives the residual (the sum of the
    streams) after every layer."""
    eps = float(cfg["norm"]["eps"])
    W = {k: v.float() for k, v in tensors.items()}
    x = W["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    x = layer_norm(x, W["embed.norm"], W["embed.norm.b"], eps)
    hyper = cfg.get("streams") is not None          # hyper-connections also with a single stream
    S = int(cfg["streams"]) if hyper else 1
    xs = [x.clone() for _ in range(S)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        subs = [(1, lambda hn, L=layer, pre=pre: MIXERS[L["type"]](hn, sub(W, pre + "mix."), L["mixer"], eps, rnd))]
        if layer.get("mlp"):
            subs.append((2, lambda hn, L=layer, pre=pre: moe_ff(hn, sub(W, pre + "mlp."), L["mlp"], rnd)))
        for qn, fn in subs:
            nw, nb = W[f"{pre}norm{qn}"], W[f"{pre}norm{qn}.b"]
            if not hyper:
                xs[0] = xs[0] + fn(rnd(layer_norm(xs[0], nw, nb, eps)))
                continue
            a_in, a_out, a_mix = W[f"{pre}hc{qn}.in"], W[f"{pre}hc{qn}.out"], W[f"{pre}hc{qn}.mix"]
            u = sum(a_in[s] * xs[s] for s in range(S))
            y = fn(rnd(layer_norm(u, nw, nb, eps)))
            xs = [sum(a_mix[s, t] * xs[s] for s in range(S)) + a_out[t] * y for t in range(S)]
        if layer_sums is not None:
            layer_sums.append(sum(xs))
    x = sum(xs)
    hn = rnd(layer_norm(x, W["final.norm"], W["final.norm.b"], eps))
    z = lin(hn, W["head"])
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * torch.tanh(z / float(cap))
    return z
