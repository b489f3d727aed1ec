"""safetensors reading/writing, binding by name, the one error for a wrong folder, random weights."""
import json
import os
import shutil

import pytest
import torch

from neurogrid_b200.config import config_from_dict
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.weights import (SafetensorsError, WeightError, index_model_dir, load_weights, read_header,
                                    write_file, write_random_model)
from tiny_configs import TINY_A, TINY_B


def test_written_file_is_read_by_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file
    t = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(2, 2, 2), "d": torch.randn(4).half()}
    p = str(tmp_path / "x.safetensors")
    write_file(p, t, {"k": "v"})
    back = load_file(p)
    for k in t:
        assert torch.equal(back[k], t[k]) and back[k].dtype == t[k].dtype
    hdr = read_header(p)
    assert hdr["a.weight"].shape == (3, 5) and hdr["a.weight"].dtype == torch.bfloat16


def test_reader_reads_what_the_safetensors_package_wrote(tmp_path):
    from safetensors.torch import save_file
    from neurogrid_b200.weights.safetensors_io import MappedFiles
    t = {"w": torch.randn(6, 4).bfloat16(), "i": torch.arange(5, dtype=torch.int64)}
    p = str(tmp_path / "model.safetensors")
    save_file(t, p)
    e = index_model_dir(str(tmp_path))
    f = MappedFiles()
    assert torch.equal(f.read(e["w"]), t["w"]) and torch.equal(f.read(e["i"]), t["i"])
    f.close()


def test_random_model_folder_loads_and_keeps_dtypes(tmp_path):
    d = write_random_model(TINY_B, 1, str(tmp_path / "m"))
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    decls = declare_tensors(config_from_dict(json.load(open(os.path.join(d, "config.json")))).model_spec())
    w = load_weights(d, decls)
    assert set(w) == set(decls)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    # same seed, same model; another seed, another model
    w2 = load_weights(write_random_model(TINY_B, 1, str(tmp_path / "m2")), decls)
    w3 = load_weights(write_random_model(TINY_B, 2, str(tmp_path / "m3")), decls)
    assert all(torch.equal(w[k], w2[k]) for k in w)
    assert any(not torch.equal(w[k], w3[k]) for k in w)
    # distributions: matrices ~N(0, .02), conv kernels ~N(0, .2), norms ~1 + N(0, .1)
    assert abs(float(w["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    assert abs(float(w["model.layers.1.conv.conv.weight"].float().std()) - 0.2) < 0.05
    nw = torch.cat([v.float() for k, v in w.items() if k.endswith("norm.weight")])
    assert abs(float(nw.mean()) - 1.0) < 0.03 and abs(float(nw.std()) - 0.1) < 0.03


def test_stored_32_bit_stays_32_bit_and_integers_become_int32(tmp_path):
    from neurogrid_b200.weights import TensorDecl
    write_file(str(tmp_path / "model.safetensors"),
               {"f": torch.randn(3), "h": torch.randn(3).half(), "b": torch.randn(3).bfloat16(),
                "i": torch.arange(3, dtype=torch.int64)})
    w = load_weights(str(tmp_path), {"f": TensorDecl((3,)), "h": TensorDecl((3,)), "b": TensorDecl((3,)),
                                     "i": TensorDecl((3,), integer=True)})
    assert (w["f"].dtype, w["h"].dtype, w["b"].dtype, w["i"].dtype) == \
        (torch.float32, torch.float32, torch.bfloat16, torch.int32)


def test_one_error_lists_everything_that_is_wrong(tmp_path):
    from safetensors.torch import load_file
    d = write_random_model(TINY_A, 0, str(tmp_path / "m"))
    t = {k: v.clone() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    del t["model.layers.2.self_attn.q_layernorm.weight"]
    del t["model.layers.0.conv.in_proj.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(2)
    t["model.layers.1.feed_forward.w2.weight"] = torch.zeros(64, 100).bfloat16()
    t["model.embedding_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_file(os.path.join(d, "model.safetensors"), t)
    decls = declare_tensors(config_from_dict(TINY_A).model_spec())
    with pytest.raises(WeightError) as e:
        load_weights(d, decls)
    err = e.value
    assert err.missing == ["model.layers.0.conv.in_proj.weight", "model.layers.2.self_attn.q_layernorm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.1.feed_forward.w2.weight"]
    assert [n for n, _, _ in err.wrong_dtype] == ["model.embedding_norm.weight"]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "expected [64, 192], file has [64, 100]", "wrong dtype"):
        assert needle in msg


def test_tied_model_rejects_a_separate_head_and_untied_needs_one(tmp_path):
    from safetensors.torch import load_file
    da = write_random_model(TINY_A, 0, str(tmp_path / "a"))
    t = {k: v.clone() for k, v in load_file(os.path.join(da, "model.safetensors")).items()}
    t["lm_head.weight"] = torch.zeros(256, 64).bfloat16()
    write_file(os.path.join(da, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_weights(da, declare_tensors(config_from_dict(TINY_A).model_spec()))
    assert e.value.unexpected == ["lm_head.weight"]
    assert "lm_head.weight" in declare_tensors(config_from_dict(TINY_B).model_spec())


def test_sharded_folder(tmp_path):
    from safetensors.torch import load_file
    d = write_random_model(TINY_A, 0, str(tmp_path / "m"))
    t = {k: v.clone() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    names = sorted(t)
    half = len(names) // 2
    os.remove(os.path.join(d, "model.safetensors"))
    write_file(os.path.join(d, "model-00001-of-00002.safetensors"), {k: t[k] for k in names[:half]})
    write_file(os.path.join(d, "model-00002-of-00002.safetensors"), {k: t[k] for k in names[half:]})
    wm = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, k in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    w = load_weights(d, declare_tensors(config_from_dict(TINY_A).model_spec()))
    assert all(torch.equal(w[k], t[k]) for k in names)


def test_corrupt_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        index_model_dir(str(tmp_path))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        index_model_dir(str(tmp_path))
    with pytest.raises(SafetensorsError):
        index_model_dir(str(tmp_path / "nothing_here"))
