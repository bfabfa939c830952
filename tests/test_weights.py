"""Safetensors by name, the random-weights mode and the one clear error (no GPU)."""
import json

import pytest
import torch

from flint_b200.engine.loading import expected_from_config, write_random_model
from flint_b200.errors import WeightError
from flint_b200.weights.loader import check_names_and_shapes, load_tensors, place
from flint_b200.weights.safetensors_io import SafetensorsFile, save_safetensors
from flint_b200.weights.sources import RandomSource, SafetensorsSource, WeightSpec
from plain_phimoe import read_safetensors
from tiny import TINY_A, TINY_B


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b.c": torch.randn(7).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int32).view(2, 3),
         "e": torch.empty(0, 4)}
    save_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == sorted(t)
    for k, v in t.items():
        got = f.read(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape) and torch.equal(got, v)
    # an independent reader agrees
    other = read_safetensors(tmp_path / "x.safetensors")
    assert all(torch.equal(other[k], v) for k, v in t.items())


def test_random_mode_writes_a_model_folder(tmp_path):
    d = write_random_model(tmp_path / "m", TINY_B, seed=5, dtype=torch.bfloat16)
    assert json.loads((d / "config.json").read_text())["hidden_size"] == 96
    src = SafetensorsSource(d)
    _, expected = expected_from_config(TINY_B)
    check_names_and_shapes(src, expected)
    assert set(src.names()) == set(expected)
    assert src.dtype("layers.0.self_attn.q_proj.weight") == torch.bfloat16
    # same seed, same bits; other seed, other bits; norm scales near one, weights near zero
    d2 = write_random_model(tmp_path / "m2", TINY_B, seed=5, dtype=torch.bfloat16)
    d3 = write_random_model(tmp_path / "m3", TINY_B, seed=6, dtype=torch.bfloat16)
    a, b, c = (SafetensorsSource(x).read("layers.1.block_sparse_moe.experts.3.w2.weight") for x in (d, d2, d3))
    assert torch.equal(a, b) and not torch.equal(a, c)
    g = src.read("layers.2.input_layernorm.weight").float()
    assert abs(g.mean().item() - 1) < 0.1 and 0.03 < g.std().item() < 0.2
    assert abs(a.float().std().item() - 0.02) < 0.005
    # stored names carry the customary prefix
    raw = SafetensorsFile(d / "model.safetensors").names()
    assert "model.embed_tokens.weight" in raw and "lm_head.weight" in raw


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(tmp_path / "m", TINY_A, seed=1, dtype=torch.float32)
    tensors = read_safetensors(d / "model.safetensors")
    tensors.pop("model.layers.0.self_attn.k_proj.bias")
    tensors.pop("model.norm.weight")
    tensors["model.layers.1.extra.weight"] = torch.zeros(2)
    tensors["model.layers.1.block_sparse_moe.experts.2.w1.weight"] = torch.zeros(96, 63)
    tensors["lm_head.weight"] = torch.zeros(512, 64, dtype=torch.int32)
    save_safetensors(d / "model.safetensors", tensors)
    _, expected = expected_from_config(TINY_A)
    with pytest.raises(WeightError) as e:
        load_tensors(SafetensorsSource(d), expected, "float32", "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "layers.0.self_attn.k_proj.bias" in msg and "norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "layers.1.extra.weight" in msg
    assert "wrong shapes or types (2)" in msg and "expected (96, 64), found (96, 63)" in msg and "lm_head.weight" in msg


def test_type_policy():
    m = WeightSpec((2, 2))
    v = WeightSpec((2,), role="vector")
    t = WeightSpec((2,), role="table")
    bf, f32, f16 = (torch.ones(2, 2, dtype=d) for d in (torch.bfloat16, torch.float32, torch.float16))
    assert place(bf, m, "bfloat16", "cpu").dtype == torch.bfloat16          # kept in bfloat16
    assert place(f32, m, "bfloat16", "cpu").dtype == torch.float32          # stored in 32-bit: stays so
    assert place(f16, m, "bfloat16", "cpu").dtype == torch.bfloat16
    assert place(bf, m, "float32", "cpu").dtype == torch.float32            # the 32-bit mode widens everything
    assert place(torch.ones(2, dtype=torch.bfloat16), v, "bfloat16", "cpu").dtype == torch.float32
    assert place(torch.ones(2, dtype=torch.int64), t, "bfloat16", "cpu").dtype == torch.int32


def test_bad_files(tmp_path):
    with pytest.raises(WeightError, match="neither"):
        SafetensorsSource(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsSource(tmp_path)
    (tmp_path / "model.safetensors").write_bytes((10 ** 6).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafetensorsSource(tmp_path)


def test_random_source_is_order_independent():
    specs = {"a": WeightSpec((4, 4)), "b": WeightSpec((4,), role="vector", init="gamma")}
    s1, s2 = RandomSource(specs, 3, torch.float32), RandomSource(specs, 3, torch.float32)
    b1 = s1.read("b")
    a1 = s1.read("a")
    assert torch.equal(s2.read("a"), a1) and torch.equal(s2.read("b"), b1)


def test_fused_checkpoint_tensors_are_split_by_rows(tmp_path):
    """A folder that stores q|k|v stacked as ``qkv_proj`` (weights and biases) loads to the same tensors as one
    that stores them apart; a fused tensor of the wrong shape is named in the one error."""
    d = write_random_model(tmp_path / "m", TINY_A, seed=2, dtype=torch.float32)
    _, expected, fused = expected_from_config(TINY_A, with_fused=True)
    apart = load_tensors(SafetensorsSource(d), expected, "float32", "cpu", fused)
    tensors = read_safetensors(d / "model.safetensors")
    for l in range(TINY_A["num_hidden_layers"]):
        pre = f"model.layers.{l}.self_attn."
        for kind in ("weight", "bias"):
            tensors[pre + "qkv_proj." + kind] = torch.cat([tensors.pop(pre + f"{x}_proj.{kind}") for x in "qkv"], 0)
    save_safetensors(d / "model.safetensors", tensors)
    src = SafetensorsSource(d)
    assert "layers.0.self_attn.q_proj.weight" not in src.names()
    together = load_tensors(src, expected, "float32", "cpu", fused)
    assert set(together) == set(apart) and all(torch.equal(together[k], apart[k]) for k in apart)
    # without the rule the same folder is refused, and the message names what is missing and what is unexpected
    with pytest.raises(WeightError, match="qkv_proj"):
        load_tensors(src, expected, "float32", "cpu")
    # a fused tensor with the wrong number of rows
    tensors["model.layers.1.self_attn.qkv_proj.weight"] = torch.zeros(100, 64)
    save_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_tensors(SafetensorsSource(d), expected, "float32", "cpu", fused)
    msg = str(e.value)
    assert "layers.1.self_attn.qkv_proj.weight: expected (128, 64)" in msg and "64 + 32 + 32" in msg and "found (100, 64)" in msg
    assert "layers.1.self_attn.q_proj.weight" in msg           # its pieces are reported missing


def test_fused_gate_up_of_the_dense_feed_forward():
    """The dense gated MLP takes ``gate_up_proj`` (gate rows, then up rows), as the reference's Phi loader does."""
    from flint_b200.parts.base import BuildContext
    from flint_b200.parts.ffn import GatedMLP
    from flint_b200.weights.sources import FusedView
    part = GatedMLP({"hidden_size": 8, "intermediate_size": 6}, BuildContext(None, torch.device("cpu"), "float32"))
    expected = part.weights()

    class Src:
        t = {"gate_up_proj.weight": torch.arange(96.0).view(12, 8), "down_proj.weight": torch.zeros(8, 6)}
        def names(self): return list(self.t)
        def shape(self, n): return tuple(self.t[n].shape)
        def dtype(self, n): return self.t[n].dtype
        def read(self, n, spec=None, device="cpu"): return self.t[n]
    got = load_tensors(Src(), expected, "float32", "cpu", part.fused())
    assert torch.equal(got["gate_proj.weight"], Src.t["gate_up_proj.weight"][:6])
    assert torch.equal(got["up_proj.weight"], Src.t["gate_up_proj.weight"][6:])
