"""The Sufolix configuration reader and its mapping to a model description (no GPU)."""
import copy
import json
import os

import pytest
import torch

import sufolix_cases as cases
from inferloop_b200.config import ConfigError, UnsupportedConfig, read_model_config
from inferloop_b200.models.decoder import declare_weights


def spec_of(config):
    return read_model_config(json.dumps(config))


def test_the_architecture_is_found_by_its_single_name():
    arch, cfg, spec = spec_of(cases.CONFIG_P)
    assert arch.name == "sufolix" and spec.architecture == "Sufolix"
    assert (spec.vocab_size, spec.hidden_size, spec.residual_streams) == (331, 96, 3)
    assert spec.embedding_scale == 3.0 and spec.head_name == "head" and spec.embedding_name == "embed"
    assert read_model_config(json.dumps(cases.CONFIG_R))[2].residual_streams == 1


def test_every_size_and_constant_reaches_the_parts():
    _, cfg, spec = spec_of(cases.CONFIG_P)
    kinds = [(l.block.kind, l.mixer.kind, l.feed_forward.kind) for l in spec.layers]
    assert kinds == [("hyper_connections", "gqa_attention", "swiglu"), ("hyper_connections", "gqa_attention", "routed_experts"),
                     ("hyper_connections", "gqa_attention", "none"), ("hyper_connections", "gqa_attention", "routed_experts")]
    m0, m1, m2 = (spec.layers[i].mixer for i in range(3))
    assert (m0["num_heads"], m0["num_kv_heads"], m0["head_dim"], m0["v_head_dim"], m0["scale"]) == (6, 3, 16, 24, 0.31)
    assert m0["position"].kind == "rope_interleaved" and m0["position"]["rotary_dim"] == 8 and m0["position"]["theta"] == 5000.0
    assert m1["position"].kind == "none"
    assert (m0["value_mix"], m1["value_mix"], m2["value_mix"]) == ("first", None, "mixed")    # the first that mixes keeps, later ones mix
    assert m0["qk_norm"] == "unweighted" and m0["qk_norm_after_rotation"] and m0["bias"] == "qkv" and m0["qk_norm_eps"] == 2e-5
    f1, f3 = spec.layers[1].feed_forward, spec.layers[3].feed_forward
    assert (f1["experts"], f1["top_k"], f1["expert_inter"], f1["shared_inter"], f1["shared_gate"]) == (5, 2, 24, 40, True)
    assert (f3["experts"], f3["top_k"], f3["expert_inter"], f3["shared_inter"], f3["shared_gate"]) == (4, 3, 40, 0, False)
    assert f1["score"] == "sigmoid" and f1["weight_on"] == "input" and not f1["renormalize"]
    assert spec_of(cases.CONFIG_R)[2].layers[0].block.kind == "pre_norm"


def test_declared_tensors_have_the_file_names_and_shapes():
    decls = {d.name: d for d in declare_weights(spec_of(cases.CONFIG_P)[2])}
    assert decls["embed"].shape == (331, 96) and decls["head"].shape == (331, 96) and decls["final.norm"].shape == (96,)
    assert decls["l0.mix.q"].shape == (96, 96) and decls["l0.mix.k"].shape == (48, 96) and decls["l0.mix.v"].shape == (72, 96)
    assert decls["l0.mix.o"].shape == (96, 144) and decls["l0.mix.v.b"].shape == (72,) and "l0.mix.o.b" not in decls
    assert decls["l2.mix.vmix"].shape == () and not decls["l2.mix.vmix"].optional
    assert decls["l0.mix.vmix"].optional and decls["l1.mix.vmix"].optional        # stored or not, never read
    assert decls["l0.hc1.mix"].shape == (3, 3) and decls["l0.hc2.in"].shape == (3,) and decls["l0.norm2"].shape == (96,)
    assert decls["l2.norm2"].optional and decls["l2.hc2.out"].optional and "l2.mlp.gate" not in decls
    assert decls["l1.mlp.router"].shape == (5, 96) and decls["l1.mlp.e4.down"].shape == (96, 24)
    assert decls["l1.mlp.shared.sg"].shape == (1, 96) and decls["l1.mlp.shared.up"].shape == (40, 96)
    assert "l3.mlp.shared.sg" not in decls and "l3.mlp.e3.gate" in decls and "l3.mlp.e4.gate" not in decls
    plain_names = {d.name for d in declare_weights(spec_of(cases.CONFIG_R)[2])}
    assert not any(".hc" in n for n in plain_names)


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu2"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 5), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), ConfigError),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), ConfigError),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), ConfigError),          # mixing layers must agree
    (lambda c: c.__setitem__("streams", 0), ConfigError),
    (lambda c: c.__setitem__("streams", 17), ConfigError),
    (lambda c: c.pop("vocab"), ConfigError),
    (lambda c: c["norm"].__setitem__("eps", 0), ConfigError),
    (lambda c: c.__setitem__("layers", []), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), ConfigError),
])
def test_what_the_reader_refuses(change, error):
    c = copy.deepcopy(cases.CONFIG_P)
    change(c)
    with pytest.raises(error):
        spec_of(c)


def test_a_random_folder_round_trips_and_optional_tensors_may_be_left_out(tmp_path):
    from inferloop_b200.weights import write_random_model
    from inferloop_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    path = write_random_model(str(tmp_path / "m"), cases.CONFIG_S, 3, torch.bfloat16, prefix="")
    f = SafetensorsFile(os.path.join(path, "model.safetensors"))
    names = f.names()
    assert "l1.mix.vmix" in names and f.tensor("l1.mix.vmix").shape == ()
    assert 0.0 < float(f.tensor("l1.mix.vmix")) < 1.0
    assert "l0.mix.vmix" in names          # the first mixing layer's coefficient is written although nobody reads it
    keep = [(n, f.tensor(n).clone()) for n in names if n != "l0.mix.vmix"]
    f.close()
    write_safetensors(os.path.join(path, "model.safetensors"), keep)
    from inferloop_b200.weights import load_weights
    spec = spec_of(cases.CONFIG_S)[2]
    tensors, ignored = load_weights(path, declare_weights(spec), spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")
    assert "l0.mix.vmix" not in tensors and "l1.mix.vmix" in tensors and not ignored
    assert tensors["l1.hc1.mix"].dtype == torch.float32 and tensors["l1.mix.q"].dtype == torch.float32


def test_the_command_line_writes_and_inspects_a_sufolix_folder(tmp_path):
    import subprocess
    import sys
    from helpers import ROOT
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(cases.CONFIG_S))
    infer = os.path.join(ROOT, "bin", "infer")
    out = subprocess.run([sys.executable, infer, "write-random-model", "--config", str(cfg), "--seed", "4", "--out", str(tmp_path / "m")],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    out = subprocess.run([sys.executable, infer, "inspect-model", str(tmp_path / "m")], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout)
    assert info["architecture"] == "sufolix" and info["config"]["streams"] == 4
    assert [l["feed_forward"] for l in info["layers"]] == ["routed_experts", "swiglu"]
    assert [l["block"] for l in info["layers"]] == ["hyper_connections"] * 2
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    assert "embed" in SafetensorsFile(str(tmp_path / "m" / "model.safetensors")).names()      # no prefix for this architecture
