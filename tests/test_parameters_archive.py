"""tnsr's parameter archive (src/parameters.rs, docs/parameter-archive.md) in Python."""
import json
import os

import numpy as np
import pytest

from tests.helpers import kv_model
from tnsr_b200.nn import TnsrError, model_parameters
from tnsr_b200.parameters import NamedParameters, gpt_from_named, load_gpt, save_gpt


def test_named_parameter_roundtrip(tmp_path):
    named = NamedParameters()
    named.insert("policy.weight", [1.0, -2.5, 3.25, 4.0], [2, 2], "policy")
    named.insert("a.bias", [0.5], [1], "value")
    named.save(str(tmp_path), {"layers": 1})
    manifest = json.load(open(tmp_path / "manifest.json"))
    assert manifest["version"] == 1 and manifest["dtype"] == "f32-le" and manifest["data_file"] == "weights.f32"
    assert [t["name"] for t in manifest["tensors"]] == ["a.bias", "policy.weight"]          # name order
    assert [t["offset"] for t in manifest["tensors"]] == [0, 1] and manifest["tensors"][1]["count"] == 4
    assert (tmp_path / "weights.f32").read_bytes() == np.asarray([0.5, 1.0, -2.5, 3.25, 4.0], "<f4").tobytes()
    assert not (tmp_path / "weights.f32.tmp").exists() and not (tmp_path / "manifest.json.tmp").exists()
    loaded, config = NamedParameters.load(str(tmp_path))
    assert config == {"layers": 1}
    assert loaded.get("policy.weight", [2, 2]).values().tolist() == [1.0, -2.5, 3.25, 4.0]
    with pytest.raises(TnsrError):
        loaded.get("policy.weight", [4])
    with pytest.raises(TnsrError):
        loaded.get("missing", [1])
    loaded.validate_names({"a.bias", "policy.weight"})
    with pytest.raises(TnsrError):
        loaded.validate_names({"a.bias"})


def test_insert_and_load_validation(tmp_path):
    named = NamedParameters()
    named.insert("w", [1.0, 2.0], [2], "g")
    for args in (("w", [1.0], [1], "g"), ("", [1.0], [1], "g"), ("x", [1.0], [2], "g"), ("y", [float("nan")], [1], "g"),
                 ("z", [1.0], [1], "")):
        with pytest.raises(TnsrError):
            named.insert(*args)
    named.save(str(tmp_path), None)
    path = tmp_path / "manifest.json"
    good = json.load(open(path))

    def broken(**changes):
        m = json.loads(json.dumps(good))
        m.update(changes)
        json.dump(m, open(path, "w"))
        with pytest.raises(TnsrError):
            NamedParameters.load(str(tmp_path))

    broken(version=2)
    broken(dtype="f16-le")
    broken(data_file="../weights.f32")
    broken(extra=1)
    broken(tensors=[dict(good["tensors"][0], offset=1)])
    broken(tensors=[dict(good["tensors"][0], count=3)])
    broken(tensors=[dict(good["tensors"][0], shape=[1], count=1)])      # trailing data
    json.dump(good, open(path, "w"))
    (tmp_path / "weights.f32").write_bytes(np.asarray([1.0, 2.0], "<f4").tobytes() + b"\x00")
    with pytest.raises(TnsrError):
        NamedParameters.load(str(tmp_path))


@pytest.mark.parametrize("activation", ["relu", "swiglu"])
def test_gpt_archive_roundtrip(tmp_path, activation):
    model = kv_model(6, activation=activation)
    weights = model.token_embedding.values()
    weights[3] = 0.125
    model.token_embedding.set_values(weights)
    save_gpt(model, str(tmp_path))
    restored = load_gpt(str(tmp_path))
    assert restored.config() == model.config()
    for a, b in zip(model_parameters(model), model_parameters(restored)):
        assert a.shape == b.shape
        assert np.array_equal(a.values().view(np.uint32), b.values().view(np.uint32))
    named, config = NamedParameters.load(str(tmp_path))
    config["num_layers"] = 3
    with pytest.raises(TnsrError):
        gpt_from_named(named, config)


@pytest.mark.parametrize("variant", ["tiny", "tiny-separate"])
def test_reference_written_archives_reload_and_resave_byte_for_byte(tmp_path, variant):
    """The archives tnsr's own forty_five example ships (examples/forty_five/fixtures/*, written by the Rust
    `NamedParameters::save`, src/parameters.rs:100-210): loading one and saving it again must reproduce both files
    exactly -- same tensor order, offsets, JSON layout and f32 bytes -- so archives pass between the two sides."""
    src = os.path.join(os.path.dirname(__file__), "golden", "forty_five", variant)
    named, config = NamedParameters.load(src)
    assert config["token_dim"] == 8 and config["use_swiglu"] is True
    named.save(str(tmp_path), config)
    for name in ("manifest.json", "weights.f32"):
        assert (tmp_path / name).read_bytes() == open(os.path.join(src, name), "rb").read(), name
