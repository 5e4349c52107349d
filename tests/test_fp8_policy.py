"""The loader of the reference's FP8 precision policy schema (src/model/quantization.rs:44-68): a document in
that schema loads unchanged, malformed documents are refused, and the enabled set of the promoted policy is the one
the model scaffolding uses by default."""
import json

import pytest

from lfm25_inference_b200 import fp8_policy


def scale(clip):
    return {"clip_amax": clip, "quantize_multiplier": 448.0 / clip, "dequantize_multiplier": clip / 448.0}


def site(name, enabled, activation=2.0, weight=0.25):
    return {"site": name, "enabled": enabled, "activation_strategy": "amax", "weight_strategy": "amax",
            "activation_scale": scale(activation), "weight_scale": scale(weight), "local_nrmse": 0.02,
            "local_cosine": 0.999, "expected_decode_saving_us": 10.0}


def document():
    gate_up = (2, 3, 5, 7, 8, 9, 11, 15)
    down = (6, 8, 9, 10, 12, 14, 15)
    sites = []
    for layer in range(16):
        sites.append(site(f"layers.{layer}.mlp.gate_up", layer in gate_up, activation=2.0 + layer))
        sites.append(site(f"layers.{layer}.mlp.down", layer in down))
        sites.append(site(f"layers.{layer}.operator.output", False))
    sites.append(site("lm_head", True, activation=9.5))
    return {"schema_version": 1, "name": "policy_frontier_16", "source": "synthetic", "decode_only": True,
            "sites": sites}


def test_document_in_the_reference_schema_loads(tmp_path):
    path = tmp_path / "policy.json"
    path.write_text(json.dumps(document()))
    policy = fp8_policy.load_fp8_policy(str(path))
    assert policy.name == "policy_frontier_16" and policy.decode_only
    assert len(policy.enabled_sites()) == 16
    assert policy.layers_with("gate_up") == (2, 3, 5, 7, 8, 9, 11, 15)
    assert policy.layers_with("down") == (6, 8, 9, 10, 12, 14, 15)
    assert policy.lm_head_enabled()
    entry = policy.site("layers.5.mlp.gate_up")
    assert entry.activation_scale.clip_amax == 7.0
    assert entry.activation_scale.quantize_multiplier == pytest.approx(448.0 / 7.0)
    assert policy.site("layers.99.mlp.down") is None


def test_default_sites_of_the_model_are_the_promoted_policy():
    from lfm25_inference_b200 import model
    policy = fp8_policy.parse_fp8_policy(document())
    assert policy.layers_with("gate_up") == model.FP8_GATE_UP_LAYERS
    assert policy.layers_with("down") == model.FP8_DOWN_LAYERS


@pytest.mark.parametrize("damage", ["version", "no_sites", "duplicate", "enabled", "scale", "negative"])
def test_malformed_documents_are_refused(damage):
    doc = document()
    if damage == "version":
        doc["schema_version"] = 2
    elif damage == "no_sites":
        del doc["sites"]
    elif damage == "duplicate":
        doc["sites"].append(doc["sites"][0])
    elif damage == "enabled":
        doc["sites"][0]["enabled"] = "yes"
    elif damage == "scale":
        del doc["sites"][0]["weight_scale"]["clip_amax"]
    elif damage == "negative":
        doc["sites"][0]["activation_scale"]["quantize_multiplier"] = -1.0
    with pytest.raises(ValueError):
        fp8_policy.parse_fp8_policy(doc)
