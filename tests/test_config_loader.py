import json
import os

import pytest

from VAR_Q.config_loader import VARQConfig, load_varq_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG_DIR = os.path.join(ROOT, "var-q_b200", "VAR_Q")                  # this build's own configurations
REF_CFG_DIR = os.path.join(ROOT, "tests", "golden", "reference_configs")   # the reference's shipped files, as fixtures


def test_reference_shaped_files_load():
    c = load_varq_config(os.path.join(REF_CFG_DIR, "VAR-VAR_Q-8.json"))
    assert c.is_var_model() and not c.is_infinity_model()
    q = c.get_quantization_config()
    assert (q["enable"], q["q_bits"], q["quant_method"], q["qkv_format"]) == (True, 8, "G_SCALE_HEAD_DIM", "BLHc")
    assert c.get_checkpoint_paths(16)[1].endswith("var_d16.pth")
    assert c.get_inference_config()["top_k"] == 600 and c.get_batch_processing_config()["batch_size"] == 50
    i = load_varq_config(os.path.join(REF_CFG_DIR, "Infinity-VAR_Q-8.json"))
    assert i.is_infinity_model() and i.get_checkpoint_paths()[1].endswith("infinity_2b_reg.pth")
    raw = load_varq_config(os.path.join(REF_CFG_DIR, "VAR-raw.json"))
    assert raw.get_quantizer_kwargs("k") is None
    assert c.get_device() in ("cpu", "cuda")


def test_sections_are_copies_and_updates_merge(tmp_path):
    c = VARQConfig(os.path.join(REF_CFG_DIR, "VAR-VAR_Q-8.json"))
    c.get_quantization_config()["q_bits"] = 2
    assert c.get_quantization_config()["q_bits"] == 8
    c.update_config({"quantization": {"q_bits": 4}, "extra": {"a": {"b": 1}}})
    assert c.get_quantization_config()["q_bits"] == 4 and c.get_quantization_config()["quant_method"] == "G_SCALE_HEAD_DIM"
    out = tmp_path / "saved.json"
    c.save_config(str(out))
    assert json.load(open(out))["extra"]["a"]["b"] == 1
    with pytest.raises(FileNotFoundError):
        VARQConfig()            # like the reference, the default path has no file behind it


def test_per_tensor_overrides_and_aliases():
    c = load_varq_config(os.path.join(CFG_DIR, "VAR-d30-int4-asym.json"))
    k, v = c.get_quantizer_kwargs("k"), c.get_quantizer_kwargs("v")
    assert k == {"quant_bits": 4, "quant_method": "G_SCALE_HEAD_DIM", "qkv_format": "BLHc", "symmetric": False}
    assert v["quant_method"] == "G_TOKEN_HEAD" and v["group_size"] == 64 and v["symmetric"] is False
    i = load_varq_config(os.path.join(CFG_DIR, "Infinity-2b-k4-v2-group32.json"))
    assert i.get_quantizer_kwargs("k")["quant_bits"] == 4 and i.get_quantizer_kwargs("v")["quant_bits"] == 2
    with pytest.raises(ValueError):
        c.get_checkpoint_paths()
