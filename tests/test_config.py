"""Configuration and registry (no GPU)."""
import json

import pytest

from hos_b200 import models  # noqa: F401
from hos_b200.config import Gemma2Config
from hos_b200.errors import MissingMetaError, SpecError, UnsupportedArchError
from hos_b200.config.base import LayerCall, ModelPlan, PartSpec
from hos_b200.registry import config_from_dict, plan_for, registered_architectures, resolve_architecture
from helpers import TINY_A, TINY_B


def test_reads_every_key():
    cfg = config_from_dict(TINY_B)
    assert isinstance(cfg, Gemma2Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (3, 96, 6, 1, 32, 160, 512)
    assert cfg.rope_theta == 1e6 and cfg.sliding_window == 16 and cfg.rms_norm_eps == 1e-5
    assert cfg.query_pre_attn_scalar == 24 and cfg.attn_logit_softcapping == 20.0
    assert cfg.final_logit_softcapping == 15.0 and cfg.eos_token_id == (1, 7)


def test_defaults_follow_the_reference():
    raw = dict(architectures=["Gemma2ForCausalLM"], hidden_size=64, num_hidden_layers=1,
               num_attention_heads=4, intermediate_size=32, vocab_size=10)
    cfg = config_from_dict(raw)
    assert cfg.num_key_value_heads == 4            # defaults to the head count
    assert cfg.head_dim == 16                      # hidden / heads
    assert cfg.max_position_embeddings == 2048 and cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0
    assert cfg.query_pre_attn_scalar == 16.0       # head_dim: the reference's 1/sqrt(head_dim)
    assert cfg.attn_logit_softcapping == 0.0 and cfg.final_logit_softcapping == 0.0
    assert cfg.sliding_window == 4096 and cfg.eos_token_id == ()


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_required_key_is_named(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(MissingMetaError, match=key):
        config_from_dict(raw)


def test_wrong_type_and_bad_values():
    with pytest.raises(MissingMetaError, match="hidden_size"):
        config_from_dict(dict(TINY_A, hidden_size="64"))
    with pytest.raises(MissingMetaError, match="multiple"):
        config_from_dict(dict(TINY_A, num_attention_heads=5))
    with pytest.raises(MissingMetaError, match="even"):
        config_from_dict(dict(TINY_A, head_dim=15))
    with pytest.raises(MissingMetaError, match="rms_norm_eps"):
        config_from_dict(dict(TINY_A, rms_norm_eps=0.0))


def test_unknown_architecture_lists_the_registered_ones():
    with pytest.raises(UnsupportedArchError) as e:
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"], model_type="llama"))
    assert "LlamaForCausalLM" in str(e.value) and "Gemma2ForCausalLM" in str(e.value)
    assert "Gemma2ForCausalLM" in registered_architectures()


def test_model_type_is_a_fallback():
    raw = dict(TINY_A)
    del raw["architectures"]
    assert resolve_architecture(raw) == "Gemma2ForCausalLM"


def test_config_round_trips_through_json():
    cfg = config_from_dict(TINY_B)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


def test_plan_takes_every_number_from_the_config():
    for raw in (TINY_A, TINY_B):
        cfg = config_from_dict(raw)
        plan = plan_for(cfg)
        assert len(plan.layers) == cfg.num_hidden_layers == len(plan.schedule)
        assert plan.vocab_size == cfg.vocab_size and plan.width == cfg.hidden_size
        for l, layer in enumerate(plan.layers):
            m = layer.mixer.params
            assert m["window"] == (cfg.sliding_window if l % 2 == 0 else None)
            assert m["scale"] == pytest.approx(cfg.query_pre_attn_scalar ** -0.5)
            assert (m["n_heads"], m["n_kv_heads"], m["head_dim"]) == (
                cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
            assert m["softcap"] == cfg.attn_logit_softcapping
            assert m["position"].params["theta"] == cfg.rope_theta
            assert layer.feed_forward.params["inner"] == cfg.intermediate_size
            assert set(layer.norms) == {"pre_mixer", "post_mixer", "pre_ffn", "post_ffn"}
            assert all(n.params["eps"] == cfg.rms_norm_eps and n.params["add_one"] for n in layer.norms.values())
        assert plan.head.params["softcap"] == cfg.final_logit_softcapping
        assert plan.embedding.params["scale"] == pytest.approx(cfg.hidden_size ** 0.5)
        assert plan.stop_token_ids == cfg.eos_token_id


def test_plan_validation_rejects_bad_run_orders():
    plan = plan_for(config_from_dict(TINY_A))
    bad = ModelPlan(plan.width, plan.vocab_size, plan.max_positions, plan.embedding, plan.layers,
                    [LayerCall(0), LayerCall(5)], plan.final_norm, plan.head)
    with pytest.raises(SpecError, match="layer 5"):
        bad.validate()
    bad.schedule = [LayerCall(0, cache_from=0)]
    with pytest.raises(SpecError, match="does not run before"):
        bad.validate()
    bad.schedule = [LayerCall(0), LayerCall(1, cache_from=0), LayerCall(0, cache_from=1)]
    with pytest.raises(SpecError, match="no cache of its own"):
        bad.validate()


def test_registry_finds_the_packages_own_parts_whatever_was_imported_first():
    """In a fresh interpreter that imported nothing but the registry: a built-in part, the built-in architecture and
    the list of architectures are there (the tables fill themselves on the first look-up)."""
    import os
    import subprocess
    import sys
    code = ("from hos_b200.registry import part_impl, registered_architectures, config_from_dict\n"
            "assert part_impl('norm', 'rmsnorm').__name__ == 'RMSNorm'\n"
            "assert 'Gemma2ForCausalLM' in registered_architectures()\n"
            "print('ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-c", code], cwd=root, stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=300)
    assert p.returncode == 0 and p.stdout.decode().strip() == "ok", p.stderr.decode()[-2000:]
