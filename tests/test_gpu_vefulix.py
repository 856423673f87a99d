"""The Vefulix design in the engine against the plain statement of its equations
(`tests/plain/vefulix_plain.py`): each mechanism alone, then whole models under every way of cutting
the work: whole prompts, tokens one by one through the state and the cache, batches of unequal
requests through slots and pages that are used again, long decoding, and greedy generation through
the session.  Sizes differ from test to test (also sizes that are 1 or equal to one another), and
where random weights would hide a fault the weights are edited so that it shows."""
import functools
import json
import os

import pytest
import torch

from helpers import plain_weights, prompts_for
from plain import vefulix_plain as P

pytestmark = pytest.mark.gpu

MLSTM = {"heads": 2, "dim": 24, "vdim": 40, "gate_cap": 12.0}
DELTA = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4}
LATENT = {"heads": 3, "dim": 16, "vdim": 24, "q_rank": 40, "kv_rank": 56, "scale": 0.2}
MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 40}}


def compare(got, ref, dtype, what=""):
    """float32: every logit within 3e-3 (absolute + relative): summation orders and exp / tanh
    implementations differ, and sharpened softmaxes and recurrences carry that on, while a fault of the
    state, the cache or the batch moves logits by tenths.
    bfloat16: both sides round activations to bfloat16 but not at exactly the same places, so a token whose
    router logits nearly tie may choose another expert on one side; such a token is off by a good part of an
    expert's output, and what follows it in a recurrent state a little.  So rows are judged one by one: the
    root-mean-square error of a row against the largest logit must be below 1.2 % for all but 15 % of the rows
    (at least two; a recurrent state carries one token's other expert on for a few tokens), below 0.6 % for the
    median row, and below 30 % for every row (the plain implementation run with and without its
    bfloat16 roundings differs from itself by as much).  A fault hits most rows."""
    got, ref = torch.as_tensor(got).float().cpu(), torch.as_tensor(ref).float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    if dtype == "float32":
        bad = err > 3e-3 + 3e-3 * ref.abs()
        assert not bad.any(), (f"{what}: {int(bad.sum())} of {err.numel()} values differ, first at "
                               f"{torch.nonzero(bad)[0].tolist()}; max abs err {err.max().item():.3g}")
        return
    rows = err.pow(2).mean(-1).sqrt() / ref.abs().max()
    over = int((rows > 0.012).sum())
    assert rows.max() < 0.3, f"{what}: row {int(rows.argmax())} is off by {rows.max().item():.3g} of the largest logit"
    assert over <= max(2, int(0.15 * len(rows))), f"{what}: {over} of {len(rows)} rows are off (worst {rows.max().item():.3g})"
    assert len(rows) < 8 or rows.median() < 0.006, f"{what}: the median row is off by {rows.median().item():.3g}"


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": dict(mixer), "mlp": None if mlp is None else json.loads(json.dumps(mlp))}


def config(layers, width=64, vocab=96, streams=None, softcap=None, eps=1e-5):
    cfg = {"architecture": "Vefulix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


FULL = config([layer("latent_attention", LATENT, MOE), layer("delta", DELTA, MOE), layer("mlstm", MLSTM, MOE),
               layer("latent_attention", dict(LATENT, heads=2, dim=24, vdim=16, kv_rank=24, scale=0.35)),
               layer("delta", dict(DELTA, heads=2, kv_heads=2, dim=40, vdim=16, conv=2), MOE)],
              width=72, vocab=200, streams=2, softcap=9.0)
# the same mechanisms at sizes the tensor-core products and the 16-byte accesses do not take (a width of 50)
ODD = config([layer("mlstm", dict(MLSTM, heads=3, dim=20, vdim=12), dict(MOE, router={"experts": 3, "top": 3})),
              layer("latent_attention", dict(LATENT, heads=1, dim=12, vdim=20, q_rank=12, kv_rank=20), MOE),
              layer("delta", dict(DELTA, heads=1, kv_heads=1, dim=12, vdim=12, conv=1),
                    {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 4, "top": 1}})],
             width=50, vocab=77, streams=3, softcap=30.0, eps=1e-6)
PLAIN_RESIDUAL = config([layer("delta", DELTA, MOE), layer("latent_attention", LATENT, MOE), layer("mlstm", MLSTM)],
                        width=64, vocab=128)


def sharpen(tensors):
    """Queries and keys of the attention layers larger, so that the softmax stands on few keys and one
    wrong or missing key moves the logits; sinks made to matter."""
    for name in list(tensors):
        if name.endswith(".mix.uq") or name.endswith(".mix.uk"):
            tensors[name] = tensors[name] * 2.0
        if name.endswith(".mix.sink"):
            tensors[name] = tensors[name] * 0 + torch.linspace(0.5, 2.5, tensors[name].numel()).to(tensors[name].dtype)


def make_model(root, cfg, seed, dtype, edit=None, std=0.1):
    """A folder with seeded random weights for `cfg` (edited by `edit`), loaded by the engine, and the same
    tensors widened to float32 for the plain implementation."""
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
    return str(tmp_path_factory.mktemp("vefulix"))


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


ALONE = {
    "mlstm": [layer("mlstm", MLSTM)],
    "delta": [layer("delta", DELTA)],
    "delta_one_group": [layer("delta", dict(DELTA, heads=3, kv_heads=1, dim=32, vdim=8, conv=3))],
    "latent_attention": [layer("latent_attention", LATENT)],
    "latent_equal_sizes": [layer("latent_attention", dict(LATENT, heads=2, dim=32, vdim=32, q_rank=32, kv_rank=32))],
    "latent_twenty_heads": [layer("latent_attention", dict(LATENT, heads=20, dim=32, vdim=32, q_rank=24, kv_rank=64, scale=0.18))],
    "latent_forty_heads_tcgen05": [layer("latent_attention", dict(LATENT, heads=40, dim=64, vdim=64, q_rank=72, kv_rank=128, scale=0.12))],
    "latent_rank_32": [layer("latent_attention", dict(LATENT, heads=5, dim=16, vdim=48, q_rank=16, kv_rank=32))],
    "moe": [layer("mlstm", MLSTM, MOE)],
    "moe_every_expert": [layer("mlstm", MLSTM, dict(MOE, router={"experts": 3, "top": 3}))],
    "moe_one_expert_no_shared": [layer("mlstm", MLSTM, {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 6, "top": 1}})],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(root, name, dtype):
    cfg = config(ALONE[name])
    model, weights = make_model(root, cfg, 3, dtype, sharpen)
    eng = engine_of(model)
    for n, prompt in zip((1, 2, 5, 37, 130), prompts_for({"vocab_size": cfg["vocab"]}, (1, 2, 5, 37, 130), seed=1)):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {n} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams", [1, 2, 4])
def test_residual_streams(root, streams, dtype):
    """Hyper-connections with one stream still mix and scale (they are not the plain residual)."""
    cfg = config([layer("delta", DELTA, MOE), layer("mlstm", MLSTM)], streams=streams)
    model, weights = make_model(root, cfg, 5, dtype)
    prompt = prompts_for({"vocab_size": cfg["vocab"]}, (23,), seed=2)[0]
    compare(run_whole(engine_of(model), prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{streams} streams")


def test_soft_cap_and_its_absence(root):
    for cap in (None, 2.0):
        cfg = config([layer("mlstm", MLSTM)], softcap=cap)
        model, weights = make_model(root, cfg, 6, "float32", std=0.3)
        prompt = prompts_for({"vocab_size": cfg["vocab"]}, (9,), seed=3)[0]
        ref = P.forward(cfg, weights, prompt)
        assert cap is None or ref.abs().max() > 0.5 * cap          # the cap bends these logits
        compare(run_whole(engine_of(model), prompt), ref, "float32", f"cap {cap}")


WHOLE_MODELS = {"full": FULL, "odd": ODD, "plain_residual": PLAIN_RESIDUAL}
LENGTHS = (1, 3, 63, 64, 65, 129, 200)


@functools.lru_cache(maxsize=None)
def _setup(root, name, dtype):
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 11, dtype, sharpen)
    prompts = prompts_for({"vocab_size": cfg["vocab"]}, LENGTHS, seed=7)
    return model, prompts, [P.forward(cfg, weights, p, rounding(dtype)) for p in prompts]


CASES = [(n, d) for n in sorted(WHOLE_MODELS) for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts(root, name, dtype):
    model, prompts, want = _setup(root, name, dtype)
    eng = engine_of(model)
    for p, ref in zip(prompts, want):
        compare(run_whole(eng, p), ref, dtype, f"{name}: {len(p)} tokens whole")
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_tokens_one_by_one(root, name, dtype):
    """The state and the cache carry a sequence: prompts cut at several places (down to one token of
    prompt), the rest decoded one by one, across page borders of the latent cache."""
    model, prompts, want = _setup(root, name, dtype)
    eng = engine_of(model)
    for p, ref in zip(prompts, want):
        for head in sorted({1, len(p) // 2, max(1, len(p) - 40)}):
            if head < 1 or (head >= len(p) and len(p) > 1):
                continue
            slot = eng.open_sequence()
            rows = [eng.step([(slot, p[:head])], want="all")]
            for t in p[head:]:
                rows.append(eng.step([(slot, [t])], want="last"))
            eng.check_device()
            compare(torch.cat(rows), ref, dtype, f"{name}: {len(p)} tokens, {head} as prompt")
            eng.close_sequence(slot)
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_through_slots_and_pages_used_again(root, name, dtype):
    """Batches of unequal requests (a one-token prompt among them) in a cache with 3 slots; shorter
    requests end earlier; the next batch takes the slots, pages and state the last one gave back."""
    model, prompts, want = _setup(root, name, dtype)
    eng = engine_of(model, max_tokens=64 * 8, max_sequences=3)
    order = [[0, 4, 5], [6, 1], [2, 3, 0], [5, 6]]
    for batch in order:
        cut = {i: max(1, len(prompts[i]) - 7 - 3 * k) for k, i in enumerate(batch)}
        slots = {i: eng.open_sequence() for i in batch}
        rows = {i: [] for i in batch}
        got = eng.step([(slots[i], prompts[i][:cut[i]]) for i in batch], want="all")
        at = 0
        for i in batch:
            rows[i].append(got[at:at + cut[i]])
            at += cut[i]
        live = [i for i in batch if cut[i] < len(prompts[i])]
        for i in batch:
            if i not in live:
                eng.close_sequence(slots[i])
        while live:
            got = eng.step([(slots[i], [prompts[i][cut[i]]]) for i in live], want="last")
            for k, i in enumerate(live):
                rows[i].append(got[k:k + 1])
                cut[i] += 1
            for i in [i for i in live if cut[i] == len(prompts[i])]:
                eng.close_sequence(slots[i])
                live.remove(i)
        eng.check_device()
        for i in batch:
            compare(torch.cat(rows[i]), want[i], dtype, f"{name}: request {i} in batch {batch}")
    eng.cache.check()
    assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(root, dtype):
    """A short prompt and 300 tokens one by one: recurrent state and the growing latent cache."""
    model, _, _ = _setup(root, "full", dtype)
    cfg = WHOLE_MODELS["full"]
    _, weights = make_model(root, cfg, 11, dtype, sharpen)
    p = prompts_for({"vocab_size": cfg["vocab"]}, (303,), seed=9)[0]
    ref = P.forward(cfg, weights, p, rounding(dtype))
    eng = engine_of(model)
    slot = eng.open_sequence()
    rows = [eng.step([(slot, p[:3])], want="all")] + [eng.step([(slot, [t])], want="last") for t in p[3:]]
    eng.check_device()
    compare(torch.cat(rows), ref, dtype, "300 tokens decoded")


def test_a_far_key_and_the_sink_decide(root):
    """Attention made to stand on single keys: with sharpened queries and keys the plain implementation
    itself changes visibly when the first key is hidden or the sink is left out, so the comparison above
    would see either fault."""
    cfg = config([layer("latent_attention", LATENT)])
    _, weights = make_model(root, cfg, 3, "float32", sharpen)
    p = prompts_for({"vocab_size": cfg["vocab"]}, (130,), seed=1)[0]
    ref = P.forward(cfg, weights, p)
    no_sink = dict(weights)
    no_sink["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -1e9)
    assert (P.forward(cfg, no_sink, p) - ref).abs().max() > 1e-2
    assert (P.forward(cfg, weights, p[1:])[-1] - ref[-1]).abs().max() > 1e-3


@pytest.mark.parametrize("name", ["full", "plain_residual"])
def test_greedy_generation_through_the_session(root, name):
    """`generate` (the scheduler's batches, the sampler, steps fed from device memory) against greedy
    choices made from the plain implementation's logits."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 11, "float32", sharpen)
    prompts = prompts_for({"vocab_size": cfg["vocab"]}, (1, 6, 70, 17), seed=4)
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


def test_command_line_and_random_folder(root, capsys):
    from inference_engine_rust_b200 import cli
    cfg = config([layer("delta", DELTA, MOE), layer("latent_attention", LATENT)], streams=2, softcap=5.0)
    path = os.path.join(root, "cfg.json")
    with open(path, "w") as f:
        json.dump(cfg, f)
    out = os.path.join(root, "cli_model")
    assert cli.main(["random-model", "--config", path, "--seed", "2", "--out", out]) == 0
    capsys.readouterr()
    assert cli.main(["-m", out, "-n", "5", "--stop-token", "-1", "3 9 27"]) == 0
    ids = capsys.readouterr().out.split()
    assert len([t for t in ids if t.lstrip("-").isdigit()]) >= 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(root, tmp_path, dtype):
    """bin/trace_run picks the architecture from config.json: requests whole, with their last tokens one by one,
    and as unequal batches whose shorter requests end earlier; every wanted row against the plain implementation."""
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import write_random_model
    import test_gpu_trace_run as R
    cfg = WHOLE_MODELS["full"]
    vocab = cfg["vocab"]
    folder = str(tmp_path / "model")
    write_random_model(folder, cfg, seed=13, dtype=dtype, std=0.1)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    sharpen(tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    weights = plain_weights(folder)
    prompts = prompts_for({"vocab_size": vocab}, (1, 33, 64, 140), seed=2)
    want = [P.forward(cfg, weights, p, rounding(dtype)) for p in prompts]

    out = str(tmp_path / "whole")
    R.replay(folder, dtype, R.whole_trace(prompts), out, max_tokens=192)
    for i in range(len(prompts)):
        compare(R.read(out, i, vocab), want[i], dtype, f"whole, request {i}")

    out = str(tmp_path / "tail")
    steps, where = R.tail_trace(prompts)
    R.replay(folder, dtype, steps, out, max_tokens=192)
    for i in range(len(prompts)):
        compare(torch.cat([R.read(out, s, vocab) for s in where[i]]), want[i], dtype, f"last tokens one by one, request {i}")

    out = str(tmp_path / "batch")
    tails = {i: min(t, len(prompts[i]) - 1) for i, t in {0: 0, 1: 9, 2: 3, 3: 17}.items()}
    steps, rows = R.batch_trace(prompts, [[3, 0, 1], [2, 1]], tails)
    R.replay(folder, dtype, steps, out, max_tokens=320)
    files = {}
    for i in (0, 2, 3):
        got = []
        for s, r in rows[i]:
            if s not in files:
                files[s] = R.read(out, s, vocab)
            got.append(files[s][r])
        compare(torch.stack(got), want[i], dtype, f"unequal batches, request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_replayed_as_graphs(root, dtype):
    """Short prompt steps that want their last rows are captured into a CUDA graph from a shape bucket's
    second use on (padding tokens and padding sequences inside): same logits as the first, eager, run, also
    with state and pages used again in between."""
    model, prompts, want = _setup(root, "full", dtype)
    eng = engine_of(model, max_tokens=64 * 8, max_sequences=4)
    batches = [[1, 0], [1, 2], [0, 1], [2, 1], [1]]                  # lengths 3, 1, 63: buckets of 16 and 64 tokens
    for turn, batch in enumerate(batches * 2):
        slots = [eng.open_sequence() for _ in batch]
        got = eng.step([(s, prompts[i]) for s, i in zip(slots, batch)], want="last")
        more = eng.step([(s, [prompts[3][len(prompts[i])]]) for s, i in zip(slots, batch)], want="last")   # and one token each
        eng.check_device()
        for k, i in enumerate(batch):
            compare(got[k:k + 1], want[i][-1:], dtype, f"turn {turn}: last row of a {len(prompts[i])}-token prompt")
        assert torch.isfinite(more).all()
        for s in slots:
            eng.close_sequence(s)
    assert any(isinstance(k, tuple) and k and k[0] == "prompt" for k in eng._graphs), "no prompt step was replayed"


@pytest.mark.parametrize("lanes", [1, 2, 8, 16])
def test_recurrences_with_every_split_of_the_state(root, lanes, monkeypatch):
    """The recurrent kernels keep a column of the state in 1 to 32 lanes, chosen per launch by the step's parallelism
    (a tiny model always gets 32); forced here so that every variant is compared, in prompts and in decoding."""
    monkeypatch.setenv("IERT_RECURRENT_LANES", str(lanes))
    cfg = config([layer("delta", dict(DELTA, heads=2, kv_heads=1, dim=32, vdim=40, conv=3)),
                  layer("mlstm", dict(MLSTM, heads=3, dim=24, vdim=72))], width=64, vocab=64)
    model, weights = make_model(root, cfg, 17, "float32")
    prompts = prompts_for({"vocab_size": cfg["vocab"]}, (70, 9, 31), seed=8)
    eng = engine_of(model)
    slots = [eng.open_sequence() for _ in prompts]
    rows = [[] for _ in prompts]
    got = eng.step([(s, p[:-5]) for s, p in zip(slots, prompts)], want="all")
    at = 0
    for i, p in enumerate(prompts):
        rows[i].append(got[at:at + len(p) - 5])
        at += len(p) - 5
    for k in range(5, 0, -1):
        got = eng.step([(s, [p[-k]]) for s, p in zip(slots, prompts)], want="last")
        for i in range(len(prompts)):
            rows[i].append(got[i:i + 1])
    eng.check_device()
    for i, p in enumerate(prompts):
        compare(torch.cat(rows[i]), P.forward(cfg, weights, p), "float32", f"{lanes} lanes per column, request {i}")
