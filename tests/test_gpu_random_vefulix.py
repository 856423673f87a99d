"""Vefulix configurations drawn at random (layer order, every size, streams, soft cap, experts), each run as
one batch of unequal prompts whose last tokens are decoded together, in 32-bit and in bfloat16, against the plain
implementation.  IERT_TEST_RANDOM_VEFULIX=N draws N configurations instead of six (50 others were run once: none differed)."""
import os
import random

import pytest
import torch

import test_gpu_vefulix as T
from helpers import prompts_for
from plain import vefulix_plain as P

pytestmark = pytest.mark.gpu

COUNT = int(os.environ.get("IERT_TEST_RANDOM_VEFULIX", "6"))


def draw_layer(rng):
    kind = rng.choice(["mlstm", "delta", "latent_attention"])
    if kind == "mlstm":
        m = {"heads": rng.choice([1, 2, 4, 6]), "dim": rng.choice([16, 32, 48, 64, 96]), "vdim": rng.choice([16, 32, 64, 128]),
             "gate_cap": rng.choice([8.0, 15.0, 30.0])}
    elif kind == "delta":
        kv = rng.choice([1, 2])
        m = {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": rng.choice([16, 32, 64, 128]),
             "vdim": rng.choice([16, 32, 64, 96]), "conv": rng.choice([2, 3, 4, 5])}
    else:
        d = rng.choice([16, 32, 48, 64, 128])
        m = {"heads": rng.choice([1, 2, 4, 8]), "dim": d, "vdim": rng.choice([d, d, 32, 64]), "q_rank": rng.choice([32, 48, 96, 128]),
             "kv_rank": rng.choice([32, 64, 96, 128, 160, 72]), "scale": round(d ** -0.5 * rng.choice([1.0, 0.5, 2.0]), 4)}
    mlp = None
    if rng.random() < 0.8:
        mlp = {"kind": "moe", "expert": {"ff": rng.choice([16, 32, 64, 96])},
               "router": {"experts": rng.choice([4, 8, 16, 24]), "top": rng.choice([1, 2, 3, 4])}}
        if rng.random() < 0.7:
            mlp["shared"] = {"ff": rng.choice([32, 64, 128])}
    return T.layer(kind, m, mlp)


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("random_vefulix"))


@pytest.mark.parametrize("case", range(COUNT))
def test_random_configuration(root, case):
    rng = random.Random(1000 + case)
    cfg = T.config([draw_layer(rng) for _ in range(rng.choice([2, 3, 4, 5]))], width=rng.choice([128, 192, 256, 320, 384]),
                   vocab=rng.choice([256, 500, 1000]), streams=rng.choice([None, 1, 2, 3, 4]),
                   softcap=rng.choice([None, 10.0, 30.0]), eps=rng.choice([1e-5, 1e-6]))
    prompts = prompts_for({"vocab_size": cfg["vocab"]}, (1, rng.randint(2, 60), rng.randint(61, 140), rng.randint(141, 330)), seed=case)
    for dtype in ("float32", "bfloat16"):
        model, weights = T.make_model(root, cfg, 100 + case, dtype, T.sharpen, std=0.06)
        want = [P.forward(cfg, weights, p, T.rounding(dtype)) for p in prompts]
        eng = T.engine_of(model, max_tokens=64 * 12, max_sequences=4)
        slots = [eng.open_sequence() for _ in prompts]
        tails = [min(len(p) - 1, 6 + 9 * i) for i, p in enumerate(prompts)]
        rows = [[] for _ in prompts]
        got, at = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all"), 0
        for i, (p, t) in enumerate(zip(prompts, tails)):
            rows[i].append(got[at:at + len(p) - t])
            at += len(p) - t
        pos = [len(p) - t for p, t in zip(prompts, tails)]
        live = [i for i in range(len(prompts)) if pos[i] < len(prompts[i])]
        for i in range(len(prompts)):
            if i not in live:
                eng.close_sequence(slots[i])
        while live:
            got = eng.step([(slots[i], [prompts[i][pos[i]]]) for i in live], want="last")
            for k, i in enumerate(live):
                rows[i].append(got[k:k + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(prompts[i])]:
                eng.close_sequence(slots[i])
                live.remove(i)
        eng.check_device()
        for i in range(len(prompts)):
            T.compare(torch.cat(rows[i]), want[i], dtype, f"case {case} ({dtype}), request {i}: {cfg}")
