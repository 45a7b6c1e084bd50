"""Safetensors reading and writing, the one error for weights that do not fit, random folders (CPU)."""
import json
import os
import struct

import pytest
import torch

import cbis_b200 as cb
import plain_gpt
import tiny_configs as tc
from cbis_b200.models import Model, load_model
from cbis_b200.weights import read_model_tensors, read_safetensors, write_safetensors


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    back = read_safetensors(p)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    try:
        from safetensors.torch import load_file
    except ImportError:
        return
    lib = load_file(p)
    assert all(torch.equal(lib[k], t[k]) for k in t)


def test_stored_forms(tmp_path):
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"),
                      {"transformer.x": torch.randn(4).half(), "y": torch.randn(4), "z": torch.arange(4),
                       "w": torch.randn(4).to(torch.bfloat16)})
    got = read_model_tensors(str(tmp_path / "m"))
    assert got["x"].dtype == torch.bfloat16 and got["w"].dtype == torch.bfloat16   # 16-bit floats are kept as bfloat16
    assert got["y"].dtype == torch.float32                                          # stored in 32-bit: stays so
    assert got["z"].dtype == torch.int32                                            # integer tables


def test_random_folder_is_reproducible_and_readable(folder_b, tmp_path):
    cfg = cb.load_config(folder_b)
    other = str(tmp_path / "again")
    cb.write_model_folder(other, cfg, seed=12, scheme=cb.InitScheme(*tc.INIT_B))
    a, b = read_model_tensors(folder_b), read_model_tensors(other)
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    cb.write_model_folder(other, cfg, seed=13, scheme=cb.InitScheme(*tc.INIT_B))
    assert not torch.equal(read_model_tensors(other)["wte.weight"], a["wte.weight"])
    pc, pw = plain_gpt.read_model_folder(folder_b, torch.float32)          # the tests' own reader agrees
    assert all(torch.equal(pw[k], a[k].float()) for k in a)
    assert a["wte.weight"].dtype == torch.bfloat16
    assert abs(a["h.0.attn.c_attn.weight"].float().std().item() - 0.05) < 0.005
    assert abs(a["h.1.ln_1.weight"].float().mean().item() - 1.0) < 0.05
    assert "lm_head.weight" in a and pc["n_inner"] == 320


def test_one_error_lists_everything(folder_a, tmp_path):
    t = read_model_tensors(folder_a)
    del t["h.1.ln_2.bias"], t["wpe.weight"]
    t["h.0.attn.c_proj.weight"] = torch.zeros(64, 63)
    t["h.0.mlp.c_fc.bias"] = torch.zeros(255)
    t["h.9.extra"] = torch.zeros(1)
    t["h.0.attn.bias"] = torch.zeros(1, 1, 8, 8)           # a buffer GPT-2 files carry: ignored
    t["lm_head.weight"] = torch.zeros(256, 64)             # tied model: ignored
    d = str(tmp_path / "bad")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(tc.TINY_A, f)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(cb.WeightsError) as e:
        load_model(d, "float32", "cpu")
    msg = str(e.value)
    assert "missing tensors (2): h.1.ln_2.bias, wpe.weight" in msg
    assert "unexpected tensors (1): h.9.extra" in msg
    assert "h.0.attn.c_proj.weight: stored (64, 63), model needs (64, 64)" in msg
    assert "h.0.mlp.c_fc.bias: stored (255,), model needs (256,)" in msg
    assert "attn.bias" not in msg and "lm_head" not in msg


def test_untied_model_needs_its_head(folder_b, tmp_path):
    t = read_model_tensors(folder_b)
    del t["lm_head.weight"]
    d = str(tmp_path / "nohead")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(tc.TINY_B, f)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(cb.WeightsError, match=r"missing tensors \(1\): lm_head.weight"):
        load_model(d, "float32", "cpu")


def test_broken_files(tmp_path):
    p = str(tmp_path / "model.safetensors")
    with pytest.raises(cb.WeightsError, match="does not exist"):
        read_safetensors(p)
    open(p, "wb").write(b"abc")
    with pytest.raises(cb.WeightsError, match="too short"):
        read_safetensors(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(cb.WeightsError, match="header length"):
        read_safetensors(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]},
                      "u": {"dtype": "Q7", "shape": [1], "data_offsets": [0, 1]},
                      "v": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(cb.WeightsError) as e:
        read_safetensors(p)
    assert "t: data_offsets" in str(e.value) and "u: unknown dtype" in str(e.value) and "v: 8 bytes stored" in str(e.value)


def test_loaded_dtypes_by_role(folder_b):
    m32 = load_model(folder_b, "float32", "cpu")
    m16 = load_model(folder_b, "bfloat16", "cpu")
    a32, a16 = m32.layers[0].mixer, m16.layers[0].mixer
    assert a32.w_qkv.dtype == torch.float32 and a16.w_qkv.dtype == torch.bfloat16
    assert a32.b_qkv.dtype == torch.float32 and a16.b_qkv.dtype == torch.float32      # vectors act in 32-bit
    assert m16.token_table.dtype == torch.bfloat16 and m16.head is not m16.token_table
    assert load_model.__module__ and Model is not None


def test_random_weights_are_drawn_by_declared_role_not_by_name():
    """A norm's scale is drawn around 1 because its declaration says so, whatever it is called; a tensor whose
    name merely looks like a norm's is drawn as its role says."""
    from cbis_b200.weights import InitScheme, TensorDecl, random_tensors
    decls = [TensorDecl("rms.scale", (64,), "norm_weight"), TensorDecl("rms.shift", (64,), "norm_bias"),
             TensorDecl("h.0.ln_1.weight", (64, 64), "matrix"), TensorDecl("out.bias", (64,), "vector")]
    t = random_tensors(decls, 3, InitScheme(0.02, 0.5, 0.1, 0.3), torch.float32)
    assert abs(t["rms.scale"].mean().item() - 1.0) < 0.05 and 0.05 < t["rms.scale"].std().item() < 0.2
    assert abs(t["rms.shift"].mean().item()) < 0.15 and 0.15 < t["rms.shift"].std().item() < 0.5
    assert abs(t["h.0.ln_1.weight"].mean().item()) < 0.01 and t["h.0.ln_1.weight"].std().item() < 0.03
    assert 0.3 < t["out.bias"].std().item() < 0.7
    plain = random_tensors(decls[:1], 3, InitScheme(), torch.float32)
    assert torch.equal(plain["rms.scale"], torch.ones(64))
    with pytest.raises(ValueError, match="role"):
        TensorDecl("x", (1,), "gamma")


def test_head_and_embedding_are_parts_of_the_spec():
    """A tensor name stands for a plain token table or an untied plain head; a PartSpec names any other kind."""
    from cbis_b200.config import PartSpec
    spec = cb.config_from_dict(tc.TINY_B).model_spec()
    assert spec.embedding_spec() == PartSpec("token_table", {"vocab_size": 317, "width": 96, "tensor": "wte.weight"})
    assert spec.head_spec().params["tensor"] == "lm_head.weight"
    m = Model(spec)
    names = [d.name for d in m.declared()]
    assert names[0] == "wte.weight" and names[-1] == "lm_head.weight" and len(names) == len(set(names))
    tied = Model(cb.config_from_dict(tc.TINY_A).model_spec())
    assert "lm_head.weight" not in [d.name for d in tied.declared()]


def test_sizes_no_kernel_takes_are_refused_when_the_model_is_built():
    big_head = dict(tc.TINY_A, n_embd=1040, n_head=2)                 # head size 520
    with pytest.raises(ValueError, match="head_dim=520"):
        Model(cb.config_from_dict(big_head).model_spec())
    wide = dict(tc.TINY_A, n_embd=65536, n_head=512)
    with pytest.raises(ValueError, match="width 65536"):
        Model(cb.config_from_dict(wide).model_spec())
