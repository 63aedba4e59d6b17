"""Configuration and registry (no GPU)."""
import json

import pytest

import qstream_b200 as qs
from qstream_b200.config import architecture_names, config_from_dict, load_config
from util import TINY_A, TINY_B


def test_reads_gptj_keys_and_derives_sizes():
    cfg = config_from_dict({**TINY_A, "architectures": ["GPTJForCausalLM"]})
    assert isinstance(cfg, qs.GptjConfig)
    assert (cfg.head_dim, cfg.inner, cfg.rotary) == (16, 256, 8)
    cfg = config_from_dict({**TINY_B, "model_type": "gptj"})           # the alias
    assert (cfg.head_dim, cfg.inner, cfg.rotary, cfg.activation_function) == (32, 320, 32, "gelu")
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.names["q"] == "transformer.h.1.attn.q_proj.weight"
    assert spec.layers[0].norms["input"].eps == 1e-6
    assert spec.head.bias and not spec.head.tied


def test_defaults():
    cfg = config_from_dict(dict(architectures=["GPTJForCausalLM"], n_layer=1, n_embd=32, n_head=2,
                                n_positions=16, vocab_size=10))
    assert cfg.rotary == 16 and cfg.inner == 128 and cfg.layer_norm_epsilon == 1e-5
    assert cfg.activation_function == "gelu_new" and cfg.rope_theta == 10000.0
    assert cfg.model_spec().stop_tokens == ()
    cfg = config_from_dict(dict(architectures=["GPTJForCausalLM"], n_layer=1, n_embd=32, n_head=2,
                                n_ctx=16, vocab_size=10, eos_token_id=3))
    assert cfg.n_positions == 16 and cfg.model_spec().stop_tokens == (3,)


def test_round_trip(tmp_path):
    cfg = config_from_dict({**TINY_B, "architectures": ["GPTJForCausalLM"]})
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(tmp_path) == cfg


@pytest.mark.parametrize("change,code", [
    (dict(n_head=5), qs.QsError.INVALID_MODEL),                 # width not divisible
    (dict(rotary_dim=7), qs.QsError.INVALID_MODEL),             # odd
    (dict(rotary_dim=18), qs.QsError.INVALID_MODEL),            # wider than the head
    (dict(n_layer=0), qs.QsError.INVALID_MODEL),
    (dict(vocab_size=0), qs.QsError.INVALID_MODEL),
    (dict(n_positions=0), qs.QsError.INVALID_MODEL),
    (dict(layer_norm_epsilon=0.0), qs.QsError.INVALID_MODEL),
    (dict(n_embd="64"), qs.QsError.INVALID_MODEL),
    (dict(activation_function="swish"), qs.QsError.UNSUPPORTED_ARCH),
    (dict(tie_word_embeddings=True), qs.QsError.UNSUPPORTED_ARCH),
    (dict(eos_token_id=256), qs.QsError.INVALID_MODEL),
])
def test_bad_values(change, code):
    with pytest.raises(qs.QStreamError) as e:
        config_from_dict({**TINY_A, "architectures": ["GPTJForCausalLM"], **change})
    assert e.value.code == code


def test_missing_key_and_unknown_architecture(tmp_path):
    d = {**TINY_A, "architectures": ["GPTJForCausalLM"]}
    del d["n_embd"]
    with pytest.raises(qs.QStreamError, match="n_embd"):
        config_from_dict(d)
    with pytest.raises(qs.QStreamError) as e:
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"]})
    assert e.value.code == qs.QsError.UNSUPPORTED_ARCH and "GPTJForCausalLM" in str(e.value)
    with pytest.raises(qs.QStreamError) as e:
        config_from_dict(dict(TINY_A))
    assert e.value.code == qs.QsError.INVALID_MODEL
    with pytest.raises(qs.QStreamError) as e:
        load_config(tmp_path)
    assert e.value.code == qs.QsError.FILE_NOT_FOUND
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(qs.QStreamError) as e:
        load_config(tmp_path)
    assert e.value.code == qs.QsError.FILE_CORRUPTED


def test_registering_an_architecture():
    class OtherConfig(qs.GptjConfig):
        architecture = "OtherForCausalLM"
        model_type = "other"
    qs.register_architecture(OtherConfig, "other")
    assert "OtherForCausalLM" in architecture_names()
    cfg = config_from_dict({**TINY_A, "architectures": ["OtherForCausalLM"]})
    assert type(cfg) is OtherConfig
