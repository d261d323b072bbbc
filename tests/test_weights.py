"""Safetensors by name, the one error for what does not fit, random-weights mode (CPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from infinicore_infer_b200.config import MiniCPMConfig, read_config
from infinicore_infer_b200.parts import model_manifest
from infinicore_infer_b200.weights import (KEEP, MATRIX, TABLE, VECTOR, DictWeights, FileWeights,
                                            SafetensorsError, WeightError, check_manifest,
                                            index_directory, random_tensors, read_header, read_tensor,
                                            stored_dtype, write_file, write_model_folder)


def test_round_trip_of_every_type(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "a.f32": torch.randn(3, 5, generator=g),
        "b.bf16": torch.randn(7, generator=g).to(torch.bfloat16),
        "c.f16": torch.randn(2, 2, 2, generator=g).to(torch.float16),
        "d.i64": torch.arange(6).reshape(2, 3),
        "e.i32": torch.arange(4, dtype=torch.int32),
        "f.scalar": torch.tensor(3.5),
        "g.empty": torch.zeros(0, 4),
    }
    path = str(tmp_path / "model.safetensors")
    write_file(path, tensors, {"format": "pt"})
    header = read_header(path)
    assert set(header) == set(tensors)
    for name, t in tensors.items():
        back = read_tensor(header[name])
        assert back.dtype == t.dtype and back.shape == t.shape
        assert torch.equal(back, t)


def test_file_is_readable_by_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"x": torch.randn(4, 3).to(torch.bfloat16), "y": torch.arange(5, dtype=torch.int32)}
    path = str(tmp_path / "m.safetensors")
    write_file(path, t)
    back = st.load_file(path)
    assert all(torch.equal(back[k], v) for k, v in t.items())
    # and the other way round
    st.save_file(t, str(tmp_path / "n.safetensors"))
    h = read_header(str(tmp_path / "n.safetensors"))
    assert all(torch.equal(read_tensor(h[k]), v) for k, v in t.items())


def test_broken_files_raise(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        read_header(str(p))
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_header(str(p))
    head = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        read_header(str(p))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        index_directory(str(empty))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    spec = MiniCPMConfig.from_dict(TINY_A).model_spec()
    manifest = model_manifest(spec)
    tensors = random_tensors(manifest, seed=0)
    shapes = {n: tuple(t.shape) for n, t in tensors.items()}
    check_manifest(manifest, shapes)                       # fits
    del shapes["model.layers.1.mlp.up_proj.weight"], shapes["model.norm.weight"]
    shapes["model.layers.0.self_attn.q_proj.weight"] = (64, 32)
    shapes["model.layers.0.mlp.down_proj.weight"] = (160, 64)
    shapes["model.layers.7.extra.weight"] = (1,)
    shapes["rotary.inv_freq"] = (8,)
    with pytest.raises(WeightError) as e:
        check_manifest(manifest, shapes, where="somewhere")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight", "rotary.inv_freq"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.mlp.down_proj.weight",
                                               "model.layers.0.self_attn.q_proj.weight"]
    text = str(err)
    for word in ("missing (2)", "unexpected (2)", "wrong shape (2)", "up_proj", "rotary.inv_freq",
                 "expected [64, 64] found [64, 32]", "somewhere"):
        assert word in text


def test_output_matrix_is_optional_and_decides_tying():
    spec = MiniCPMConfig.from_dict(TINY_A).model_spec()
    manifest = model_manifest(spec)
    assert manifest["lm_head.weight"].optional
    tied = random_tensors(manifest, seed=0)
    assert "lm_head.weight" not in tied
    untied = random_tensors(manifest, seed=0, include_optional=True)
    check_manifest(manifest, {n: tuple(t.shape) for n, t in untied.items()})


def test_storage_rule():
    assert stored_dtype(torch.float16) == torch.bfloat16
    assert stored_dtype(torch.bfloat16) == torch.bfloat16
    assert stored_dtype(torch.float32) == torch.float32      # stored in 32 bits: stays so
    assert stored_dtype(torch.int64) == torch.int32
    src = {"m16": torch.randn(4, 4).to(torch.float16), "m32": torch.randn(4, 4),
           "v": torch.randn(4).to(torch.bfloat16), "t": torch.arange(4), "k32": torch.randn(3)}
    bf = DictWeights(src, torch.bfloat16, "cpu")
    assert bf.get("m16", MATRIX).dtype == torch.bfloat16
    assert bf.get("m32", MATRIX).dtype == torch.bfloat16     # operand of a 16-bit product
    assert bf.get("m16", KEEP).dtype == torch.bfloat16
    assert bf.get("k32", KEEP).dtype == torch.float32
    assert bf.get("v", VECTOR).dtype == torch.float32
    assert bf.get("t", TABLE).dtype == torch.int32
    f32 = DictWeights(src, torch.float32, "cpu")
    assert f32.get("m16", MATRIX).dtype == torch.float32
    assert f32.get("m16", KEEP).dtype == torch.float32
    assert torch.equal(f32.get("m16", MATRIX), src["m16"].float())


def test_random_mode_writes_a_loadable_folder(tmp_path):
    cfg = MiniCPMConfig.from_dict(TINY_B)
    d = write_model_folder(cfg, str(tmp_path / "m"), seed=1, std=0.03, norm_std=0.02)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert read_config(d) == cfg
    fw = FileWeights(d, torch.float32, "cpu")
    check_manifest(model_manifest(cfg.model_spec()), fw.shapes())
    assert "lm_head.weight" in fw.index                      # untied configuration
    q = fw.get("model.layers.2.self_attn.q_proj.weight")
    assert q.shape == (96, 96) and fw.index["model.layers.2.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert 0.02 < q.std() < 0.04
    n = fw.get("model.norm.weight", VECTOR)
    assert fw.index["model.norm.weight"].dtype == torch.float32 and abs(float(n.mean()) - 1) < 0.02
    # same seed, same bytes; another seed, other values
    d2 = write_model_folder(cfg, str(tmp_path / "m2"), seed=1, std=0.03, norm_std=0.02)
    assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()
    d3 = write_model_folder(cfg, str(tmp_path / "m3"), seed=2, std=0.03, norm_std=0.02)
    q3 = FileWeights(d3, torch.float32, "cpu").get("model.layers.2.self_attn.q_proj.weight")
    assert not torch.equal(q, q3)


def test_tied_folder_has_no_output_matrix(tmp_path):
    d = write_model_folder(MiniCPMConfig.from_dict(TINY_A), str(tmp_path / "a"), seed=0)
    assert "lm_head.weight" not in index_directory(d)


def test_unused_tensors_warn_and_fail_only_when_strict():
    """A checkpoint may hold more than the model reads (the reference reads every key and uses what it needs,
    scripts/jiuge.py:400-407): that is a warning naming the tensors, an error only for a strict load."""
    from infinicore_infer_b200.weights import UnusedTensorsWarning
    spec = MiniCPMConfig.from_dict(TINY_A).model_spec()
    manifest = model_manifest(spec)
    shapes = {n: tuple(t.shape) for n, t in random_tensors(manifest, seed=0).items()}
    shapes["model.layers.0.self_attn.rotary_emb.inv_freq"] = (8,)
    with pytest.warns(UnusedTensorsWarning, match="rotary_emb.inv_freq"):
        check_manifest(manifest, shapes)
    with pytest.raises(WeightError) as e:
        check_manifest(manifest, shapes, strict=True)
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and not e.value.missing


def test_fused_rows_come_out_as_one_tensor(tmp_path):
    """``get_rows`` hands a part its fused matrix: the named tensors one below the other, in the role's type."""
    import warnings
    from infinicore_infer_b200.weights import write_file
    from infinicore_infer_b200.weights.loader import Float16RoundedWarning
    a, b, c = torch.randn(4, 6), torch.randn(2, 6), torch.randn(3, 6)
    d = tmp_path / "m"
    d.mkdir()
    write_file(str(d / "model.safetensors"), {"a": a.to(torch.bfloat16), "b": b.to(torch.float16), "c": c,
                                              "v1": torch.randn(5).to(torch.bfloat16), "v2": torch.randn(3)})
    want = torch.cat([a.to(torch.bfloat16).float(), b.to(torch.float16).float(), c])
    f32 = FileWeights(str(d), torch.float32, "cpu")
    assert torch.equal(f32.get_rows(["a", "b", "c"], MATRIX), want)            # widened exactly
    bf = FileWeights(str(d), torch.bfloat16, "cpu")
    with pytest.warns(Float16RoundedWarning, match="float16"):
        got = bf.get_rows(["a", "b", "c"], MATRIX)
    assert got.dtype == torch.bfloat16 and torch.equal(got, want.to(torch.bfloat16))
    with warnings.catch_warnings():
        warnings.simplefilter("error")                                          # said once per source
        bf.get("b", MATRIX)
    v = bf.get_rows(["v1", "v2"], VECTOR)
    assert v.dtype == torch.float32 and v.shape == (8,)
    with pytest.raises(ValueError, match="cannot be stacked"):
        bf.get_rows(["a", "v1"], MATRIX)
    dw = DictWeights({"a": a, "b": b}, torch.float32, "cpu")
    assert torch.equal(dw.get_rows(["a", "b"]), torch.cat([a, b]))
