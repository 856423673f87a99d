"""Configuration of the Vefulix design without a device: keys, defaults, refusals, the spec it builds, the
tensors it expects, and the random-weights mode."""
import json

import pytest
import torch

from inference_engine_rust_b200 import ConfigError, config_from_dict, spec_of, write_random_model
from inference_engine_rust_b200.engine import Model
from inference_engine_rust_b200.parts.base import Runtime

MOE = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 24}}
CFG = {
    "architecture": "Vefulix", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "streams": 2, "logit_softcap": 7.5,
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "gate_cap": 10.0}, "mlp": MOE},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 4, "q_rank": 12, "kv_rank": 20, "scale": 0.3},
         "mlp": None},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "conv": 3},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 1}}},
    ],
}


def expected(cfg):
    return Model(spec_of(config_from_dict(cfg)), Runtime(dtype=torch.float32, device="cpu")).expected_tensors()


def test_the_architecture_is_found_by_its_single_name_key_and_round_trips():
    c = config_from_dict(CFG)
    assert c.architecture == "Vefulix" and c.streams == 2 and c.logit_softcap == 7.5
    assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert c.to_dict()["layers"][2]["mlp"].get("shared") is None and "shared" not in c.to_dict()["layers"][2]["mlp"]


def test_spec_follows_the_layer_list():
    spec = spec_of(config_from_dict(CFG))
    assert [l.mixer.kind for l in spec.layers] == ["mlstm", "latent_attention", "gated_delta"]
    assert [l.ffn is None for l in spec.layers] == [False, True, False]
    assert spec.residual_streams == 2 and spec.head.kind == "softcap" and spec.head["cap"] == 7.5
    assert all(l.block.kind == "hyper" and l.norm.kind == "layernorm" for l in spec.layers)
    assert spec.layers[2].ffn["shared_ff"] is None and spec.layers[0].ffn["shared_ff"] == 24


def test_without_streams_and_cap_the_plain_arrangement_and_head_are_used():
    cfg = {k: v for k, v in CFG.items() if k not in ("streams", "logit_softcap")}
    spec = spec_of(config_from_dict(cfg))
    assert spec.residual_streams is None and spec.head.kind == "linear"
    assert all(l.block.kind == "prenorm" for l in spec.layers)
    names = expected(cfg)
    assert not any(".hc" in n for n in names)


def test_expected_tensors_and_shapes():
    names = expected(CFG)
    for n, shape in {"embed": (50, 32), "embed.norm": (32,), "embed.norm.b": (32,), "final.norm.b": (32,), "head": (50, 32),
                     "l0.norm1.b": (32,), "l0.hc1.mix": (2, 2), "l0.hc2.in": (2,), "l1.hc1.out": (2,),
                     "l0.mix.i.b": (2,), "l0.mix.norm": (24,), "l0.mlp.e3.down": (32, 16), "l0.mlp.router.b": (4,),
                     "l0.mlp.shared.gate": (24, 32), "l1.mix.dkv": (20, 32), "l1.mix.uk": (16, 20), "l1.mix.uv": (8, 20),
                     "l1.mix.sink": (2,), "l2.mix.q.conv": (16, 3), "l2.mix.v.conv": (16, 3), "l2.mix.norm": (4,),
                     "l2.mix.A_log": (4,), "l2.mix.b": (4, 32)}.items():
        assert tuple(names[n].shape) == shape, n
    assert "l1.hc2.in" not in names and "l1.norm2" not in names          # a layer without a feed-forward
    assert "l2.mlp.shared.up" not in names and "l2.mlp.e3.up" not in names


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_refusals_name_the_key(edit, word):
    cfg = json.loads(json.dumps(CFG))
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_random_folder_has_every_tensor(tmp_path):
    from safetensors.torch import load_file
    write_random_model(str(tmp_path / "m"), CFG, seed=1)
    tensors = load_file(str(tmp_path / "m" / "model.safetensors"))
    assert set(tensors) == set(expected(CFG))
    mix = tensors["l0.hc1.mix"].float()
    assert (mix - torch.eye(2)).abs().max() < 0.2            # stream mixing starts near the identity
    assert json.load(open(tmp_path / "m" / "config.json"))["architecture"] == "Vefulix"
