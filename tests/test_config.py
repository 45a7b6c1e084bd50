"""Typed configuration and the architecture registry (CPU)."""
import json

import pytest

import cbis_b200 as cb
import tiny_configs as tc


def test_reads_every_size_from_config_json():
    for cfgd in (tc.TINY_A, tc.TINY_B):
        c = cb.config_from_dict(cfgd)
        for k in ("n_layer", "n_embd", "n_head", "n_inner", "n_positions", "vocab_size", "activation_function",
                  "layer_norm_epsilon", "tie_word_embeddings"):
            assert getattr(c, k) == cfgd[k]
        spec = c.model_spec()
        assert len(spec.layers) == cfgd["n_layer"] and spec.schedule == tuple(range(cfgd["n_layer"]))
        m = spec.layers[0].mixer.params
        assert m["n_head"] == cfgd["n_head"] and m["head_dim"] == cfgd["n_embd"] // cfgd["n_head"]
        assert abs(m["scale"] - (cfgd["n_embd"] // cfgd["n_head"]) ** -0.5) < 1e-12
        assert spec.layers[0].feed_forward.params["inner"] == cfgd["n_inner"]
        assert spec.layers[0].norm_mixer.params["eps"] == cfgd["layer_norm_epsilon"]
        assert (spec.head is None) == cfgd["tie_word_embeddings"]
        assert cb.config_from_dict(c.to_dict()) == c


def test_defaults_and_null_inner():
    d = dict(tc.TINY_A)
    d["n_inner"] = None
    assert cb.config_from_dict(d).n_inner == 4 * d["n_embd"]
    del d["n_inner"], d["layer_norm_epsilon"], d["tie_word_embeddings"]
    c = cb.config_from_dict(d)
    assert c.n_inner == 4 * d["n_embd"] and c.layer_norm_epsilon == 1e-5 and c.tie_word_embeddings is True


@pytest.mark.parametrize("change,word", [
    ({"n_head": 5}, "multiple"), ({"n_embd": None}, "n_embd"), ({"n_layer": 0}, "n_layer"),
    ({"activation_function": "relu"}, "activation_function"), ({"layer_norm_epsilon": 0}, "layer_norm_epsilon"),
    ({"vocab_size": "many"}, "vocab_size"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"n_inner": -3}, "n_inner"),
])
def test_bad_values_are_named(change, word):
    d = dict(tc.TINY_A)
    d.update(change)
    with pytest.raises(cb.ConfigError, match=word):
        cb.config_from_dict(d)


def test_registry_names():
    assert {"GPT2LMHeadModel", "TinyGPT"} <= set(cb.known_architectures())
    with pytest.raises(cb.ConfigError, match="unknown architecture 'LlamaForCausalLM'.*GPT2LMHeadModel"):
        cb.config_from_dict({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(cb.ConfigError, match="names no architecture"):
        cb.config_from_dict({"n_layer": 2})
    d = dict(tc.TINY_B)
    del d["architectures"]
    d["model_type"] = "gpt2"
    assert cb.config_from_dict(d).n_layer == 3


def test_load_config_from_folder(tmp_path):
    with pytest.raises(cb.ConfigError, match="does not exist"):
        cb.load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(cb.ConfigError, match="not valid JSON"):
        cb.load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tc.TINY_B))
    assert cb.load_config(str(tmp_path)).vocab_size == 317


def test_registering_another_architecture():
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec

    class TwoKinds:
        """Layers that differ, a schedule that names a layer twice, a layer that reads another's cache."""
        def __init__(self, d):
            self.d = d
        @classmethod
        def from_dict(cls, d):
            return cls(d)
        def to_dict(self):
            return self.d
        def model_spec(self):
            w = self.d["width"]
            norm = PartSpec("layernorm", {"width": w, "eps": 1e-5})
            att = lambda heads, window: PartSpec("attention", {"width": w, "n_head": heads, "n_kv_head": heads,
                                                               "head_dim": w // heads, "scale": 1.0, "window": window})
            ffn = lambda inner: PartSpec("dense", {"width": w, "inner": inner, "activation": "gelu_erf"})
            layers = (LayerSpec("h.0.", "pre_norm", att(2, 0), ffn(32), norm, norm),
                      LayerSpec("h.1.", "pre_norm", att(4, 8), ffn(48), norm, norm),
                      LayerSpec("h.2.", "pre_norm", att(2, 0), ffn(32), norm, norm, cache_source=0))
            return ModelSpec(w, 50, 64, "wte.weight", PartSpec("learned", {"width": w, "n_positions": 64}),
                             layers, (0, 1, 1, 2), norm, "ln_f.", None)

    cb.register_architecture("TwoKindsTest", TwoKinds)
    spec = cb.config_from_dict({"architectures": ["TwoKindsTest"], "width": 16}).model_spec()
    from cbis_b200.models import Model
    from cbis_b200.cache import cache_groups_of
    m = Model(spec)
    names = {t.name: t.shape for t in m.declared()}
    assert names["h.1.mlp.c_fc.weight"] == (16, 48) and names["h.0.attn.c_attn.weight"] == (16, 48)
    assert names["h.2.attn.c_attn.weight"] == (16, 16)      # reads layer 0's cache: queries only
    groups = cache_groups_of(m, 8)
    assert [g.layers for g in groups] == [[0], [1]] and [g.need.window for g in groups] == [0, 8]
