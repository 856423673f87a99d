"""The Sifasun configuration on the CPU: keys read, refusals that name the key, the spec it builds (layers that
borrow weights become schedule entries of the owner, tensor names, parts), the random folder, the cache's pair of
requests for a pair of mixers."""
import json

import pytest
import torch

from inference_engine_rust_b200.config import ConfigError, config_from_dict, preset, spec_of
from inference_engine_rust_b200.engine.model import Model
from inference_engine_rust_b200.parts.base import Runtime

ATT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "softcap": 9.0, "mask": {"size": 7},
       "rot": {"base": 1000.0, "dims": 8, "scaling": {"factor": 2.0}}}
PAIR = {"left": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 24, "scale": 0.2, "mask": {"size": 70},
                 "rot": {"base": 5000.0, "dims": 24}},
        "left_scale": 1.5, "right": {"width": 40, "blocks": 5, "conv": 3}, "right_scale": 0.5}


def cfg(layers=None, **top):
    layers = layers if layers is not None else [
        {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 48}},
        {"type": "parallel", "mixer": PAIR, "mlp": None},
        {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 48}, "weights_of": 0},
        {"type": "parallel", "mixer": PAIR, "mlp": None, "weights_of": 1}]
    d = {"architecture": "Sifasun", "vocab": 90, "width": 56, "norm": {"eps": 1e-6}, "logit_scale": 3.0,
         "layers": json.loads(json.dumps(layers))}
    d.update(top)
    return d


def test_spec_of_a_configuration():
    c = config_from_dict(cfg())
    spec = spec_of(c)
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 1] and len(spec.layers) == 2
    assert spec.head.kind == "scaled" and spec.head["scale"] == 3.0 and spec.lm_head_name is None
    assert spec.final_norm["offset"] == 1.0 and spec.layers[0].block.kind == "outnorm"
    a = spec.layers[0].mixer
    assert a.kind == "tied_kv_attention" and a["qk_norm"] == "head" and a["sink"] and a["softcap"] == 9.0 and a["window"] == 7
    assert a["position"]["freq_factors"] == [2.0] * 4 and a["position"]["rotary_dim"] == 8
    p = spec.layers[1].mixer
    assert p.kind == "parallel" and p["left"]["qk_norm"] == "whole" and not p["left"]["sink"] and p["right"].kind == "rglru"
    assert spec.layers[1].ffn is None
    model = Model(spec, Runtime(dtype=torch.float32, device="cpu"))
    names = set(model.expected_tensors())
    assert names == {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.o", "l0.mlp.gate",
                     "l0.mlp.up", "l0.mlp.down", "l1.norm1", "l1.mix.left.q", "l1.mix.left.k", "l1.mix.left.o",
                     "l1.mix.left.q.norm", "l1.mix.left.k.norm", "l1.mix.right.y", "l1.mix.right.y.b", "l1.mix.right.x",
                     "l1.mix.right.x.b", "l1.mix.right.conv", "l1.mix.right.conv.b", "l1.mix.right.ra", "l1.mix.right.ra.b",
                     "l1.mix.right.ri", "l1.mix.right.ri.b", "l1.mix.right.lam", "l1.mix.right.o"}
    assert model.expected_tensors()["l1.mix.right.ra"].shape == (5, 8, 8)
    assert config_from_dict(c.to_dict()) == c


def test_an_owner_further_down_and_names_by_place():
    layers = cfg()["layers"]
    layers = [dict(layers[0], weights_of=2), layers[1], {k: v for k, v in layers[0].items()}]
    spec = spec_of(config_from_dict(cfg(layers)))
    assert [e.layer for e in spec.schedule] == [1, 0, 1]
    assert spec.layers[1].mixer_prefix == "l2.mix." and spec.layers[0].mixer_prefix == "l1.mix."


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "mixer", "vdim"), 8, "vdim"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "right", "blocks"), 3, "blocks"),
    (("layers", 1, "type"), "mlstm", "type"), (("layers", 2, "weights_of"), 1, "weights"),
    (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"), (("norm",), None, "eps"), (("layers", 1, "mixer", "left_scale"), None, "left_scale"),
])
def test_refusals_name_the_key(path, value, word):
    raw = cfg()
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_pair_of_cache_requests():
    from inference_engine_rust_b200.cache import Cache, KVRequest, StateRequest
    reqs = {0: KVRequest(2, 16, 7), 1: (KVRequest(1, 24, 70), StateRequest((120,))), 2: KVRequest(2, 16, 7),
            3: (KVRequest(1, 24, 70), StateRequest((120,)))}
    cache = Cache(reqs, max_tokens=256, max_seq_len=256, max_sequences=3, dtype=torch.float32, device="cpu")
    kv, st = cache.layer_view(1)
    assert kv.group is cache.layer_view(3)[0].group and kv.index != cache.layer_view(3)[0].index
    assert st.state.shape == (3, 120) and cache.layer_view(0).group.req.window == 7
    s = cache.open_sequence()
    cache.reserve(s, 100)
    cache.check()
    cache.close_sequence(s)
    cache.check()


def test_presets_and_random_folder(tmp_path):
    from inference_engine_rust_b200 import write_random_model
    from inference_engine_rust_b200.weights import TensorSource
    for name in ("sifasun-tiny", "sifasun-7b-sizes"):
        spec_of(config_from_dict(preset(name)))
    d = str(tmp_path / "m")
    write_random_model(d, preset("sifasun-tiny"), seed=3)
    src = TensorSource(d)
    assert "l0.mix.right.lam" in set(src.names()) and "l4.norm1" not in set(src.names())
