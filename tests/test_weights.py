"""safetensors by name, the one error that lists what does not fit, random weights (no GPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import qstream_b200 as qs
from qstream_b200.engine.model import declared_tensors
from qstream_b200.weights import (SafetensorsFile, bind_tensors, open_checkpoint, random_tensors,
                                  write_safetensors)
import plain_gptj as P
from util import TINY, make_folder


def test_folder_round_trip_and_precision_rule(tmp_path):
    for dtype, torch_dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder, cfg = make_folder(tmp_path, "A", dtype)
        assert json.loads((folder / "config.json").read_text())["n_embd"] == 64
        files = open_checkpoint(folder)
        wanted = declared_tensors(cfg.model_spec())
        assert set(files[0].names()) == set(wanted)
        for engine_dtype in (torch.float32, torch.bfloat16):
            got = bind_tensors(files, wanted, engine_dtype, "cpu")
            # 16-bit tensors follow the engine; a tensor stored in 32-bit stays in 32-bit
            expect = torch.float32 if torch_dtype == torch.float32 else engine_dtype
            assert {t.dtype for t in got.values()} == {expect}
            assert got["transformer.wte.weight"].shape == (256, 64)
        # an independent reader sees the same numbers
        theirs = P.read_safetensors(folder / "model.safetensors")
        ours = bind_tensors(files, wanted, torch.float32, "cpu")
        for name in wanted:
            np.testing.assert_array_equal(theirs[name], ours[name].double().numpy())


def test_safetensors_package_reads_our_files(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    folder, cfg = make_folder(tmp_path, "B", "bfloat16")
    theirs = st.load_file(str(folder / "model.safetensors"))
    ours = SafetensorsFile(folder / "model.safetensors")
    assert set(theirs) == set(ours.names())
    for name, t in theirs.items():
        assert torch.equal(t, ours.read(name))
    ours_nommap = SafetensorsFile(folder / "model.safetensors", allow_mmap=False)
    assert torch.equal(ours_nommap.read("lm_head.bias"), theirs["lm_head.bias"])


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    del tensors["transformer.h.1.mlp.fc_in.bias"]
    del tensors["lm_head.bias"]
    tensors["transformer.h.0.attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["transformer.h.0.ln_1.weight"] = torch.zeros(64, dtype=torch.int32)
    tensors["transformer.extra.weight"] = torch.zeros(3)
    tensors["transformer.h.0.attn.bias"] = torch.zeros(1, 1, 8, 8)         # a buffer GPT-J files may carry
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(qs.QStreamError) as e:
        bind_tensors(open_checkpoint(folder), declared_tensors(cfg.model_spec()), torch.float32, "cpu",
                     cfg.ignored_tensor_suffixes)
    msg = str(e.value)
    assert e.value.code == qs.QsError.INVALID_MODEL
    assert "2 missing" in msg and "transformer.h.1.mlp.fc_in.bias" in msg and "lm_head.bias" in msg
    assert "1 unexpected" in msg and "transformer.extra.weight" in msg
    assert "2 wrong shape or type" in msg and "[64, 32]" in msg and "[64, 64]" in msg
    assert "transformer.h.0.attn.bias" not in msg


def test_corrupted_files(tmp_path):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    path = folder / "model.safetensors"
    raw = path.read_bytes()
    cases = {
        "truncated data": raw[:len(raw) // 2],
        "shorter than the length field": raw[:5],
        "header length beyond the file": struct.pack("<Q", 10 ** 12) + raw[8:],
        "not json": raw[:8] + b"#" + raw[9:],
    }
    for what, blob in cases.items():
        path.write_bytes(blob)
        with pytest.raises(qs.QStreamError) as e:
            SafetensorsFile(path)
        assert e.value.code == qs.QsError.FILE_CORRUPTED, what
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    header["lm_head.bias"]["data_offsets"][1] += 4          # offsets that do not match the shape
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + raw[8 + hlen:])
    with pytest.raises(qs.QStreamError, match="lm_head.bias"):
        SafetensorsFile(path)
    path.unlink()
    with pytest.raises(qs.QStreamError) as e:
        open_checkpoint(folder)
    assert e.value.code == qs.QsError.FILE_NOT_FOUND


def test_random_weights_follow_the_named_distributions():
    cfg_dict, scales, seed = TINY["B"]
    cfg = qs.GptjConfig.from_dict({**cfg_dict, "architectures": ["GPTJForCausalLM"]})
    wanted = declared_tensors(cfg.model_spec())
    a = random_tensors(wanted, seed, torch.float32, "cpu", scales)
    b = random_tensors(wanted, seed, torch.float32, "cpu", scales)
    c = random_tensors(wanted, seed + 1, torch.float32, "cpu", scales)
    assert all(torch.equal(a[n], b[n]) for n in wanted)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    w = a["transformer.h.0.mlp.fc_in.weight"]
    assert abs(w.std().item() - 0.05) < 0.003 and abs(w.mean().item()) < 0.002
    ln = a["transformer.h.2.ln_1.weight"]
    assert 0.8 <= ln.min() and ln.max() <= 1.2 and ln.std() > 0.05
    assert abs(a["lm_head.bias"].std().item() - 0.01) < 0.002
    h = random_tensors(wanted, seed, torch.bfloat16, "cpu", scales)
    assert torch.equal(h["lm_head.weight"], a["lm_head.weight"].bfloat16())   # rounded once from float32
