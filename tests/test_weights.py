"""safetensors reading/writing, name binding and its errors, random weights (no GPU)."""
import json
import os
import shutil
import struct

import pytest
import torch

import wick_b200 as wick
from wick_b200.weights.loader import check_tensors
from helpers import CONFIG_A, CONFIG_B, model_dir, tmp_root
from plain import qwen3_plain as P


def _cpu_model(cfg_json):
    cfg = wick.config_from_json(cfg_json)
    return wick.Model(wick.get_architecture(cfg.architecture).build_spec(cfg), torch.float32, "cpu")


def test_write_then_read_round_trip_all_dtypes():
    d = os.path.join(tmp_root(), "st-rt")
    os.makedirs(d, exist_ok=True)
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16),
         "i": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    wick.write_safetensors(os.path.join(d, "model.safetensors"), t)
    st = wick.SafeTensorsDir(d)
    assert sorted(st.names()) == ["a", "b", "c", "i"]
    for k, v in t.items():
        got = st.get(k).tensor()
        assert got.dtype == v.dtype and torch.equal(got, v)
    # the plain reader (an independent implementation) reads the same values
    pl = P.read_safetensors(os.path.join(d, "model.safetensors").replace("model.safetensors", "model.safetensors")) \
        if False else None
    raw = open(os.path.join(d, "model.safetensors"), "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert (8 + hlen) % 8 == 0, "data starts on an 8-byte boundary (safetensors.rs:155-158)"


def test_plain_reader_agrees_with_the_library_reader():
    d = model_dir("A")
    st = wick.SafeTensorsDir(d)
    pl = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert set(pl) == set(st.names())
    for k in pl:
        assert torch.equal(pl[k], st.get(k).tensor().float())


def test_sharded_directory():
    d = os.path.join(tmp_root(), "st-shard")
    os.makedirs(d, exist_ok=True)
    wick.write_safetensors(os.path.join(d, "s1.safetensors"), {"x": torch.ones(2)})
    wick.write_safetensors(os.path.join(d, "s2.safetensors"), {"y": torch.zeros(3)})
    json.dump({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    st = wick.SafeTensorsDir(d)
    assert sorted(st.names()) == ["x", "y"] and len(st) == 2


@pytest.mark.parametrize("blob, message", [
    (b"\x01\x02", "file too short"),
    (struct.pack("<Q", 1 << 40) + b"{}", "bad header length"),
    (struct.pack("<Q", 2) + b"[]", "header is not an object"),
    (struct.pack("<Q", 3) + b"{x}", "Expecting"),
])
def test_malformed_files(blob, message):
    d = os.path.join(tmp_root(), f"st-bad-{abs(hash(blob))}")
    os.makedirs(d, exist_ok=True)
    open(os.path.join(d, "model.safetensors"), "wb").write(blob)
    with pytest.raises(wick.SafeTensorsError, match=message):
        wick.SafeTensorsDir(d)


def test_range_and_dtype_checks():
    d = os.path.join(tmp_root(), "st-range")
    os.makedirs(d, exist_ok=True)

    def write(header):
        text = json.dumps(header).encode()
        open(os.path.join(d, "model.safetensors"), "wb").write(struct.pack("<Q", len(text)) + text + b"\0" * 16)

    write({"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}})
    with pytest.raises(wick.SafeTensorsError, match="x: data range does not match its shape"):
        wick.SafeTensorsDir(d)
    write({"x": {"dtype": "F8_E4M3", "shape": [3], "data_offsets": [0, 3]}})
    with pytest.raises(wick.SafeTensorsError, match="x: unsupported dtype F8_E4M3"):
        wick.SafeTensorsDir(d)
    write({"__metadata__": {"format": "pt"}, "x": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}})
    assert wick.SafeTensorsDir(d).get("x").shape == (2, 2)
    with pytest.raises(wick.SafeTensorsError, match="model.safetensors"):
        wick.SafeTensorsDir(os.path.join(d, "missing"))


def test_a_written_model_binds_cleanly_and_lists_every_tensor():
    for name, cfgj in (("A", CONFIG_A), ("B", CONFIG_B)):
        m = _cpu_model(cfgj)
        st = wick.SafeTensorsDir(model_dir(name))
        check_tensors(m, st)
        table = m.tensor_table()
        L = cfgj["num_hidden_layers"]
        assert len(table) == 1 + 11 * L + 1 + 1
        assert "model.layers.0.self_attn.q_norm.weight" in table and "model.norm.weight" in table
        assert table["lm_head.weight"].optional
        assert ("lm_head.weight" in st) == (not cfgj["tie_word_embeddings"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    src = model_dir("B")
    d = os.path.join(tmp_root(), "w-bad")
    shutil.rmtree(d, ignore_errors=True)
    shutil.copytree(src, d)
    st = wick.SafeTensorsDir(src)
    t = {n: st.get(n).tensor().clone() for n in st.names()}
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(5, 96, dtype=torch.bfloat16)
    t["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    t["model.layers.9.stray.weight"] = torch.zeros(1)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)      # tolerated leftover of old checkpoints
    wick.write_safetensors(os.path.join(d, "model.safetensors"), t)
    m = _cpu_model(CONFIG_B)
    with pytest.raises(wick.WeightError) as ei:
        wick.load_weights(m, d)
    e = ei.value
    msg = str(e)
    assert sorted(e.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.stray.weight"]
    assert sorted(e.wrong_shape) == ["model.layers.0.self_attn.k_proj.weight", "model.layers.2.self_attn.q_norm.weight"]
    assert "missing tensor model.norm.weight" in msg
    assert "model.layers.0.self_attn.k_proj.weight: expected shape [96, 96], found [5, 96]" in msg
    assert "unexpected tensor model.layers.9.stray.weight" in msg
    assert "2 missing, 1 unexpected, 2 of the wrong shape" in msg


def test_config_that_disagrees_with_the_tensors_fails_with_expected_shape():
    # wick tests/tiny_models.rs:134-147
    src = model_dir("A")
    d = os.path.join(tmp_root(), "w-mismatch")
    shutil.rmtree(d, ignore_errors=True)
    shutil.copytree(src, d)
    j = json.load(open(os.path.join(d, "config.json")))
    j["hidden_size"] = 96
    json.dump(j, open(os.path.join(d, "config.json"), "w"))
    cfg = wick.load_config(d)
    m = wick.Model(wick.get_architecture(cfg.architecture).build_spec(cfg), torch.float32, "cpu")
    with pytest.raises(wick.WeightError, match="expected shape"):
        wick.load_weights(m, d)


def test_dtypes_are_kept_or_widened_as_declared():
    d = os.path.join(tmp_root(), "w-dtypes")
    cfg = wick.config_from_json(CONFIG_A)
    wick.write_random_model(cfg, 3, d, dtype=torch.float16)
    for dt in (torch.bfloat16, torch.float32):
        m = wick.Model(wick.get_architecture(cfg.architecture).build_spec(cfg), dt, "cpu")
        st = wick.load_weights(m, d)
        blk = m.blocks[0]
        assert blk.mixer.qkv.weight.dtype == dt and blk.mixer.qkv.weight.shape == (64 + 2 * 32, 64)
        assert blk.mixer_norm.weight.dtype == torch.float32, "vectors are always held in 32-bit"
        assert blk.mixer.q_norm.weight.dtype == torch.float32
        src_q = st.get("model.layers.0.self_attn.q_proj.weight").tensor()
        want = src_q.float().to(dt)                      # f16 -> f32 -> bf16 (model.rs:67-71)
        assert torch.equal(blk.mixer.qkv.weight[:64], want)
        assert torch.equal(blk.mixer_norm.weight, st.get("model.layers.0.input_layernorm.weight").tensor().float())
        assert m.head.is_tied and m.head.linear.weight is m.embedding.weight


def test_head_is_tied_when_its_tensor_is_absent_even_if_the_config_says_untied():
    # model.rs:190
    src = model_dir("B")
    d = os.path.join(tmp_root(), "w-tie")
    shutil.rmtree(d, ignore_errors=True)
    shutil.copytree(src, d)
    st = wick.SafeTensorsDir(src)
    t = {n: st.get(n).tensor().clone() for n in st.names() if n != "lm_head.weight"}
    wick.write_safetensors(os.path.join(d, "model.safetensors"), t)
    m = _cpu_model(CONFIG_B)
    wick.load_weights(m, d)
    assert m.head.is_tied


def test_random_weights_are_seeded_and_shaped_by_role():
    cfg = wick.config_from_json(CONFIG_B)
    d1, d2, d3 = (os.path.join(tmp_root(), f"w-rand{i}") for i in range(3))
    wick.write_random_model(cfg, 5, d1)
    wick.write_random_model(cfg, 5, d2)
    wick.write_random_model(cfg, 6, d3)
    a, b, c = (wick.SafeTensorsDir(d) for d in (d1, d2, d3))
    for n in a.names():
        assert torch.equal(a.get(n).tensor(), b.get(n).tensor())
    assert not torch.equal(a.get("lm_head.weight").tensor(), c.get("lm_head.weight").tensor())
    w = a.get("model.layers.0.mlp.gate_proj.weight").tensor().float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    nrm = a.get("model.layers.0.input_layernorm.weight").tensor().float()
    assert abs(nrm.mean().item() - 1.0) < 0.06 and 0.03 < nrm.std().item() < 0.2
    assert json.load(open(os.path.join(d1, "config.json")))["head_dim"] == 32
