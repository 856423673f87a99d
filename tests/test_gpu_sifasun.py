"""The Sifasun design in the engine against the plain statement of its equations
(`tests/plain/sifasun_plain.py`): each mechanism alone, then whole models under every way of cutting the
work: whole prompts, tokens one by one through the cache and the state, batches of unequal requests through
slots and pages that are used again, decoding until every window has passed over decoded tokens, and greedy
generation through the session.  Sizes differ from test to test (also sizes that are 1 or equal to one
another), and where random weights would hide a fault the configuration or the weights are made so that it
shows: windows of a few keys (every key carries weight), large score scales (the softmax stands on few keys,
near or far), sinks that take a good part of the denominator."""
import functools
import json
import os

import pytest
import torch

from helpers import compare as compare_exactly, plain_weights, prompts_for
from plain import sifasun_plain as P

pytestmark = pytest.mark.gpu


def compare(got, ref, dtype, what="", slack=1.0):
    """float32: the library's bound for 32-bit runs (every logit within 2e-4, absolute + relative).
    bfloat16: both sides round activations to bfloat16, but not at exactly the same places (the engine keeps the
    projections that enter norms and the recurrence in 32-bit and rounds its attention weights), and these
    models' softmaxes are sharp on purpose, which carries a rounding of a score on.  So rows are judged one by
    one: the root-mean-square error of a row against the largest logit must be below 1.2 % for all but 15 % of
    the rows (at least two), below 0.6 % for the median row, and below 30 % for every row.  A fault of the
    cache, the state or the batch hits most rows, and every case also runs in float32.  `slack` widens the bfloat16
    bounds for models of many layer runs, whose roundings add up (measured on such a model: the engine and the plain
    statement with its bfloat16 roundings are equally far from the 32-bit result)."""
    if dtype == "float32":
        return compare_exactly(got, ref, dtype, what)
    got, ref = torch.as_tensor(got).float().cpu(), torch.as_tensor(ref).float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    rows = (got - ref).pow(2).mean(-1).sqrt() / ref.abs().max()
    over = int((rows > 0.012 * slack).sum())
    assert rows.max() < 0.3, f"{what}: row {int(rows.argmax())} is off by {rows.max().item():.3g} of the largest logit"
    assert over <= max(2, int(0.15 * len(rows))), f"{what}: {over} of {len(rows)} rows are off (worst {rows.max().item():.3g})"
    assert len(rows) < 8 or rows.median() < 0.006 * slack, f"{what}: the median row is off by {rows.median().item():.3g}"


def attn(heads=4, kv_heads=2, dim=16, window=9, scale=0.6, softcap=7.0, rot_dims=8, base=900.0, factor=3.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}}
    if factor is not None:
        m["rot"]["scaling"] = {"factor": factor}
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def pair(left=None, right=None, left_scale=1.3, right_scale=0.8):
    left = left or attn(heads=3, kv_heads=3, dim=16, window=6, scale=0.4, softcap=None, rot_dims=16, factor=None)
    return {"left": left, "left_scale": left_scale, "right": right or {"width": 48, "blocks": 3, "conv": 4},
            "right_scale": right_scale}


def layer(kind, mixer, ff=40, weights_of=None):
    out = {"type": kind, "mixer": json.loads(json.dumps(mixer)), "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(layers, width=64, vocab=96, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Sifasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": layers}


ALONE = {
    "attention": [layer("attention", attn(), ff=None)],
    "attention_no_cap_no_window": [layer("attention", attn(window=None, softcap=None, factor=None), ff=None)],
    "attention_whole_head_turns_one_kv_head": [layer("attention", attn(heads=3, kv_heads=1, dim=32, rot_dims=32, window=70), ff=None)],
    "attention_nothing_turns": [layer("attention", attn(heads=2, kv_heads=2, dim=24, rot_dims=0, window=3), ff=None)],
    "attention_tcgen05_head": [layer("attention", attn(heads=4, kv_heads=2, dim=64, rot_dims=16, window=100, scale=0.3), ff=None)],
    # a projection row of more than 48 KB in 32-bit (the preparation kernel holds it in shared memory)
    "attention_wide_projection": [layer("attention", attn(heads=40, kv_heads=10, dim=256, rot_dims=64, window=50, scale=0.05), ff=None)],
    "left_alone": [layer("parallel", pair(right_scale=0.0), ff=None)],
    "right_alone": [layer("parallel", pair(left_scale=0.0), ff=None)],
    "right_one_block_two_taps": [layer("parallel", pair(right={"width": 40, "blocks": 1, "conv": 2}, left_scale=0.0), ff=None)],
    "right_every_channel_a_block_one_tap": [layer("parallel", pair(right={"width": 24, "blocks": 24, "conv": 1}, left_scale=0.0), ff=None)],
    "right_wide_blocks": [layer("parallel", pair(right={"width": 200, "blocks": 2, "conv": 7}, left_scale=0.0), ff=None)],
    "pair": [layer("parallel", pair(), ff=None)],
    "feed_forward": [layer("attention", attn(), ff=56)],
}

FULL = config([layer("parallel", pair()), layer("attention", attn()),
               layer("attention", attn(heads=6, kv_heads=3, dim=32, window=70, scale=0.35, softcap=12.0, rot_dims=32, factor=None), ff=None),
               layer("parallel", pair(), weights_of=0), layer("attention", attn(), weights_of=1),
               layer("parallel", pair(left=attn(heads=2, kv_heads=1, dim=48, window=130, scale=0.3, softcap=None, rot_dims=24,
                                                factor=None),
                                      right={"width": 96, "blocks": 4, "conv": 3}, left_scale=0.7, right_scale=1.6), ff=88)],
              width=72, vocab=200, logit_scale=2.5)
# sizes the tensor-core products and the 16-byte accesses do not take (a width of 50, a head size of 12)
ODD = config([layer("attention", attn(heads=3, kv_heads=3, dim=12, window=5, rot_dims=4), ff=30),
              layer("parallel", pair(left=attn(heads=2, kv_heads=1, dim=20, window=11, softcap=None, rot_dims=20, factor=None),
                                     right={"width": 35, "blocks": 5, "conv": 5}), ff=None),
              layer("attention", attn(heads=3, kv_heads=3, dim=12, window=5, rot_dims=4), ff=30, weights_of=0)],
             width=50, vocab=77, eps=1e-6, logit_scale=1.0)
# head sizes the tensor-core attention kernels take (64 on tcgen05, 32 and 48 on mma.sync), widths in whole tiles
TENSOR = config([layer("attention", attn(heads=4, kv_heads=2, dim=64, window=100, scale=0.3, rot_dims=32), ff=128),
                 layer("parallel", pair(left=attn(heads=4, kv_heads=2, dim=48, window=80, scale=0.3, softcap=None, rot_dims=48,
                                                  factor=None),
                                        right={"width": 128, "blocks": 2, "conv": 4}), ff=128),
                 layer("attention", attn(heads=4, kv_heads=4, dim=32, window=40, scale=0.4, softcap=5.0, rot_dims=16), ff=None)],
                width=128, vocab=256)
# heads of 128 (tcgen05 prompt attention, decode attention with pages by TMA) and recurrence blocks of 128 channels
# (several tiles of the tensor-core gates)
WIDE_HEADS = config([layer("attention", attn(heads=4, kv_heads=2, dim=128, window=150, scale=0.2, softcap=10.0, rot_dims=64), ff=None),
                     layer("parallel", pair(left=attn(heads=2, kv_heads=1, dim=128, window=90, scale=0.15, softcap=None,
                                                      rot_dims=128, factor=None),
                                            right={"width": 256, "blocks": 2, "conv": 4}), ff=256)],
                    width=256, vocab=160)
WHOLE_MODELS = {"full": FULL, "odd": ODD, "tensor": TENSOR, "wide_heads": WIDE_HEADS}


def sharpen(tensors):
    """The weights of the norms over the whole query and key projections larger, so that the softmax of the
    attention beside the recurrence stands on few keys too (the other attention has unit heads: its sharpness
    is its scale)."""
    for name in list(tensors):
        if name.endswith(".q.norm"):
            tensors[name] = tensors[name] * 2.5


def make_model(root, cfg, seed, dtype, edit=sharpen, std=0.1):
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import LoadedModel, write_random_model
    d = os.path.join(root, f"m{abs(hash((json.dumps(cfg, sort_keys=True), seed, dtype, edit is not None))) % 10 ** 9}")
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed=seed, dtype=dtype, std=std)
        if edit is not None:
            path = os.path.join(d, "model.safetensors")
            tensors = load_file(path)
            edit(tensors)
            save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    return LoadedModel.load(d, dtype=dtype), plain_weights(d)


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("sifasun"))


def rounding(dtype):
    return P.bf16 if dtype == "bfloat16" else P.exact


def engine_of(model, max_tokens=64 * 16, **kw):
    return model.session(max_tokens=max_tokens, poison_cache=True, **kw).engine


def run_whole(eng, prompt):
    slot = eng.open_sequence()
    got = eng.step([(slot, prompt)], want="all")
    eng.check_device()
    eng.close_sequence(slot)
    return got


def tokens(cfg, lengths, seed=0):
    return prompts_for({"vocab_size": cfg["vocab"]}, lengths, seed=seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(root, name, dtype):
    cfg = config(ALONE[name])
    model, weights = make_model(root, cfg, 3, dtype)
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 2, 150), seed=1):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


def test_residual_after_every_layer(root):
    """The residual after each layer run (a layer with borrowed weights counts when it runs) against the plain statement."""
    model, weights = make_model(root, FULL, 5, "float32")
    eng = engine_of(model)
    prompt = tokens(FULL, (37,), seed=2)[0]
    want, got = [], []
    P.forward(FULL, weights, prompt, residuals=want)
    model.model.after_block = lambda pos, rows, ctx: got.append(rows[:ctx.n_tokens].clone())
    try:
        run_whole(eng, prompt)
    finally:
        model.model.after_block = None
    assert len(got) == len(want) == len(FULL["layers"])
    for i, (g, w) in enumerate(zip(got, want)):
        compare(g, w, "float32", f"residual after layer run {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_whole_prompts(root, name, dtype):
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 7, dtype)
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 3, 64, 65, 300), seed=3):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_prompt_then_tokens_one_by_one(root, name, dtype):
    """A prompt in one step, then single tokens until every window has passed over decoded tokens and a page
    border has been crossed; also from the very first token on."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 8, dtype)
    eng = engine_of(model)
    for first, total in ((1, 20), (2, 75), (61, 61 + 140)):
        seq = tokens(cfg, (total,), seed=first)[0]
        ref = P.forward(cfg, weights, seq, rounding(dtype))
        slot = eng.open_sequence()
        rows = [eng.step([(slot, seq[:first])], want="all")]
        for t in seq[first:]:
            rows.append(eng.step([(slot, [t])], want="last"))
        eng.check_device()
        eng.close_sequence(slot)
        compare(torch.cat(rows), ref, dtype, f"{name}: {first} tokens, then {total - first} one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_unequal_batches_through_slots_and_pages_used_again(root, name, dtype):
    """Batches of unequal requests decoded together, the shorter ones ending earlier, in a cache so small that
    slots and pages are handed out again (poisoned when freed): every row equals the request run alone."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 9, dtype)
    eng = engine_of(model, max_tokens=64 * 7, max_sequences=4)
    for wave, lengths in enumerate(((1, 70, 5), (130, 2, 64, 33), (3, 129))):
        seqs = tokens(cfg, [n + d for n, d in zip(lengths, (9, 3, 14, 6))], seed=10 + wave)
        refs = [P.forward(cfg, weights, s, rounding(dtype)) for s in seqs]
        slots = [eng.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lengths)], want=[[n - 1] for n in lengths])
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
        done = list(lengths)
        live = list(range(len(seqs)))
        while live:
            out = eng.step([(slots[i], [seqs[i][done[i]]]) for i in live], want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                done[i] += 1
            for i in [i for i in live if done[i] == len(seqs[i])]:
                eng.close_sequence(slots[i])
                live.remove(i)
        eng.check_device()
        for i, (s, n) in enumerate(zip(seqs, lengths)):
            compare(torch.cat(got[i]), refs[i][n - 1:], dtype, f"{name}: wave {wave}, request {i} ({n} + {len(s) - n} tokens)")
        eng.cache.check()


def plant(cfg, weights, where):
    """A copy of the plain statement's configuration with one fault planted."""
    bad = json.loads(json.dumps(cfg))
    if where == "window":
        for lay in bad["layers"]:
            m = lay["mixer"] if lay["type"] == "attention" else lay["mixer"]["left"]
            m["mask"]["size"] += 1
    return bad


def test_the_tolerances_refuse_a_window_one_key_wider(root):
    """The comparison that the other tests pass is not passed by a plain statement whose windows are one key wider."""
    for name, cfg in WHOLE_MODELS.items():
        model, weights = make_model(root, cfg, 7, "float32")
        prompt = tokens(cfg, (300,), seed=3)[0]
        got = run_whole(engine_of(model), prompt)
        with pytest.raises(AssertionError):
            compare(got, P.forward(plant(cfg, weights, "window"), weights, prompt), "float32", name)


def test_a_far_key_and_the_sink_decide(root):
    """One attention layer without a window whose scores are sharp: the last token's query is made to match the key
    of a token hundreds of positions back (a query map and an embedding row made for it, a large score scale), so that dropping that one key
    would change the result; and a model whose keys all score far below zero, so that the sink takes most of
    the denominator."""
    cfg = config([layer("attention", attn(heads=2, kv_heads=1, dim=32, window=None, scale=0.9, softcap=25.0, rot_dims=0,
                                           factor=None), ff=None)], width=64, vocab=50)

    def matched(t):
        # the query map is the key map behind a turn of the input by one place, and token 48's embedding is token
        # 49's turned the same way: the query of 49 equals the key of 48 (and not its own), and their values differ
        t["l0.mix.q"] = torch.roll(t["l0.mix.k"], 1, dims=1).repeat(2, 1).contiguous()
        t["embed"][48] = torch.roll(t["embed"][49], -1)
    model, weights = make_model(root, cfg, 13, "float32", matched)
    prompt = [min(t, 47) for t in tokens(cfg, (700,), seed=5)[0]]
    prompt[40], prompt[-1] = 48, 49
    eng = engine_of(model, max_tokens=64 * 12)
    ref = P.forward(cfg, weights, prompt)
    compare(run_whole(eng, prompt), ref, "float32", "a far key in a prompt")
    slot = eng.open_sequence()
    eng.step([(slot, prompt[:-1])], want="none")
    compare(eng.step([(slot, prompt[-1:])], want="last"), ref[-1:], "float32", "a far key from the cache")
    eng.close_sequence(slot)
    without = P.forward(cfg, weights, prompt[:40] + [47] + prompt[41:])
    assert (without[-1] - ref[-1]).abs().max() > 0.05, "the far key does not matter in this test"

    def opposed(t):
        t["l0.mix.q"] = -t["l0.mix.k"].repeat(2, 1).contiguous()          # every score negative: the sink dominates
    model, weights = make_model(root, dict(cfg, vocab=51), 14, "float32", opposed)
    prompt = [7] * 30
    ref = P.forward(dict(cfg, vocab=51), weights, prompt)
    compare(run_whole(engine_of(model), prompt), ref, "float32", "a sink that dominates")


@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_greedy_generation_through_the_session(root, name):
    """`generate` (the scheduler's batches, the sampler, steps fed from device memory) against greedy
    choices made from the plain implementation's logits."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 11, "float32")
    prompts = tokens(cfg, (1, 6, 70, 17), seed=4)
    session = model.session(max_tokens=64 * 10, max_sequences=3)
    got = session.generate(prompts, max_new_tokens=12, stop_ids=[])
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            logits = P.forward(cfg, weights, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] < 1e-3:           # a close call proves nothing either way
                break
            seq.append(int(torch.argmax(logits)))
        n = len(seq) - len(p)
        assert g[:n] == seq[len(p):], f"{name}: prompt of {len(p)} tokens"


def test_command_line_and_presets(root, capsys):
    from inference_engine_rust_b200 import cli
    path = os.path.join(root, "cfg.json")
    with open(path, "w") as f:
        json.dump(ODD, f)
    out = os.path.join(root, "cli_model")
    assert cli.main(["random-model", "--config", path, "--seed", "2", "--out", out]) == 0
    capsys.readouterr()
    assert cli.main(["-m", out, "-n", "5", "--stop-token", "-1", "3 9 27"]) == 0
    ids = capsys.readouterr().out.split()
    assert len([t for t in ids if t.lstrip("-").isdigit()]) >= 5
    assert cli.main(["--random", "sifasun-tiny", "--seed", "1", "-n", "4", "--stop-token", "-1", "5 6"]) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(root, tmp_path, dtype):
    """bin/trace_run picks the architecture from config.json: requests whole, with their last tokens one by one,
    and as unequal batches whose shorter requests end earlier; every wanted row against the plain implementation."""
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import write_random_model
    import test_gpu_trace_run as R
    cfg = TENSOR if dtype == "bfloat16" else FULL
    d = str(tmp_path / "model")
    write_random_model(d, cfg, seed=21, dtype=dtype, std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = load_file(path)
    sharpen(tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    weights = plain_weights(d)
    seqs = tokens(cfg, (90, 7, 131), seed=6)
    refs = [P.forward(cfg, weights, s, rounding(dtype)) for s in seqs]
    steps, wanted = [], []
    n = 0
    for i, s in enumerate(seqs):                       # whole; then all but five tokens and the rest one by one
        steps.append({"step": n, "entries": [{"id": f"w{i}", "tokens": s, "want": [0, len(s) - 1]}], "end": [f"w{i}"]})
        wanted.append((n, [refs[i][0], refs[i][-1]]))
        n += 1
        cut = max(1, len(s) - 5)
        steps.append({"step": n, "entries": [{"id": f"d{i}", "tokens": s[:cut], "want": []}], "end": []})
        n += 1
        for j in range(cut, len(s)):
            steps.append({"step": n, "entries": [{"id": f"d{i}", "tokens": [s[j]], "want": [0]}],
                          "end": [f"d{i}"] if j == len(s) - 1 else []})
            wanted.append((n, [refs[i][j]]))
            n += 1
    cuts = [len(s) - k for s, k in zip(seqs, (4, 2, 6))]       # together: unequal prompts, then decoded until each ends
    steps.append({"step": n, "entries": [{"id": f"t{i}", "tokens": s[:c], "want": [c - 1]} for i, (s, c) in enumerate(zip(seqs, cuts))],
                  "end": []})
    wanted.append((n, [refs[i][c - 1] for i, c in enumerate(cuts)]))
    n += 1
    pos = list(cuts)
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i, s in enumerate(seqs) if pos[i] < len(s)]
        steps.append({"step": n, "entries": [{"id": f"t{i}", "tokens": [seqs[i][pos[i]]], "want": [0]} for i in live],
                      "end": [f"t{i}" for i in live if pos[i] + 1 == len(seqs[i])]})
        wanted.append((n, [refs[i][pos[i]] for i in live]))
        for i in live:
            pos[i] += 1
        n += 1
    out = str(tmp_path / "out")
    R.replay(d, dtype, steps, out, max_tokens=64 * 9)
    for step, rows in wanted:
        compare(R.read(out, step, cfg["vocab"]), torch.stack(rows), dtype, f"step {step}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_replayed_as_graphs(root, dtype):
    """Prompt steps of up to 512 tokens that want their last rows are captured into a CUDA graph from a shape
    bucket's second use on (padding tokens and padding sequences inside; the recurrence's scan in chunks for the
    longer buckets): same logits as the plain statement on every turn, with state, slots and pages used again in
    between, and the tokens after the prompt one by one."""
    cfg = WHOLE_MODELS["tensor" if dtype == "bfloat16" else "full"]
    model, weights = make_model(root, cfg, 17, dtype)
    # memory that the graphs' own buffers will be cut from holds NaN: rows of padding tokens that nobody writes show
    junk = [torch.full((16 << 20,), float("nan"), device="cuda") for _ in range(4)]
    del junk
    prompts = tokens(cfg, (3, 1, 63, 200, 140, 331), seed=8)
    want = [P.forward(cfg, weights, p + [5, 6], rounding(dtype)) for p in prompts]
    eng = engine_of(model, max_tokens=64 * 14, max_sequences=4)
    batches = [[1, 0], [3], [1, 2], [4, 0], [5], [0, 1], [3, 1], [2, 1], [5], [4]]
    for turn, batch in enumerate(batches * 2):
        slots = [eng.open_sequence() for _ in batch]
        got = eng.step([(s, prompts[i]) for s, i in zip(slots, batch)], want="last")
        more = eng.step([(s, [5]) for s in slots], want="last")
        last = eng.step([(s, [6]) for s in slots], want="last")
        eng.check_device()
        for k, i in enumerate(batch):
            n = len(prompts[i])
            compare(torch.cat([got[k:k + 1], more[k:k + 1], last[k:k + 1]]), want[i][n - 1:], dtype,
                    f"turn {turn}: a {n}-token prompt and two tokens more")
        for s in slots:
            eng.close_sequence(s)
    assert sum(1 for k in eng._graphs if isinstance(k, tuple) and k and k[0] == "prompt") >= 4, "few prompt steps were replayed"
