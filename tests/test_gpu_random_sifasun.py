"""Sifasun configurations drawn at random (layer order, every size, windows, caps, rotation, blocks and taps of the
recurrence, layers that borrow weights, layers without a feed-forward), each run as one batch of unequal prompts whose
last tokens are decoded together, in 32-bit and in bfloat16, against the plain implementation.
IERT_TEST_RANDOM_SIFASUN=N draws N configurations instead of eight."""
import os
import random

import pytest
import torch

import test_gpu_sifasun as T
from plain import sifasun_plain as P

pytestmark = pytest.mark.gpu

COUNT = int(os.environ.get("IERT_TEST_RANDOM_SIFASUN", "8"))


def draw_attention(rng, left):
    dim = rng.choice([8, 16, 24, 32, 48, 64, 80, 96, 128, 160, 256])
    kv = rng.choice([1, 2, 3, 4])
    rot = rng.choice([0, dim // 4 * 2, dim // 2, dim]) // 2 * 2
    return T.attn(heads=kv * rng.choice([1, 2, 3, 5]), kv_heads=kv, dim=dim, window=rng.choice([None, 1, 2, 7, 33, 64, 65, 100, 200]),
                  scale=round(dim ** -0.5 * rng.choice([0.7, 1.0, 2.5]) * (1.0 if left else dim ** 0.5 * 0.15), 4),
                  softcap=None if left and rng.random() < 0.8 else rng.choice([None, 4.0, 15.0, 50.0]),
                  rot_dims=rot, base=rng.choice([100.0, 10000.0, 500000.0]), factor=rng.choice([None, 1.0, 2.0, 8.0]))


def draw_layer(rng):
    ff = rng.choice([None, 24, 64, 100, 160])
    if rng.random() < 0.5:
        return T.layer("attention", draw_attention(rng, False), ff=ff)
    blocks = rng.choice([1, 2, 3, 4, 8])
    right = {"width": blocks * rng.choice([4, 8, 12, 16, 40, 64]), "blocks": blocks, "conv": rng.choice([1, 2, 3, 4, 6])}
    return T.layer("parallel", T.pair(left=draw_attention(rng, True), right=right, left_scale=rng.choice([0.5, 1.0, 1.7]),
                                      right_scale=rng.choice([0.6, 1.0, 1.4])), ff=ff)


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("random_sifasun"))


@pytest.mark.parametrize("case", range(COUNT))
def test_random_configuration(root, case):
    rng = random.Random(2000 + case)
    own = [draw_layer(rng) for _ in range(rng.choice([1, 2, 3, 4]))]
    order = list(range(len(own))) + [rng.randrange(len(own)) for _ in range(rng.choice([0, 1, 3]))]
    rng.shuffle(order)
    layers, first = [], {}
    for j in order:                       # the first run of a drawn layer owns the weights, later runs borrow them
        if j in first:
            layers.append(dict(own[j], weights_of=first[j]))
        else:
            first[j] = len(layers)
            layers.append(dict(own[j]))
    cfg = T.config(layers, width=rng.choice([40, 64, 100, 128, 192, 256]), vocab=rng.choice([61, 256, 500]),
                   eps=rng.choice([1e-5, 1e-6]), logit_scale=rng.choice([0.5, 1.0, 3.0]))
    prompts = T.tokens(cfg, (1, rng.randint(2, 60), rng.randint(61, 140), rng.randint(141, 330)), seed=case)
    for dtype in ("float32", "bfloat16"):
        model, weights = T.make_model(root, cfg, 100 + case, dtype, T.sharpen, std=0.08)
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
            T.compare(torch.cat(rows[i]), want[i], dtype, f"case {case} ({dtype}), request {i}: {cfg}",
                      slack=max(1.0, len(layers) / 5))
