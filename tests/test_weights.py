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


def test_random_weights_are_a_function_of_seed_name_and_index():
    """Counter-based: a tensor depends on the seed and its own name only, and any slice can be made alone."""
    from qstream_b200.weights.loader import TensorDecl
    from qstream_b200.weights.random_init import host_values, tensor_key
    one = random_tensors({"a.weight": TensorDecl((40, 50))}, 5, torch.float32, "cpu")
    two = random_tensors({"zzz": TensorDecl((3,), "bias"), "a.weight": TensorDecl((40, 50))}, 5, torch.float32, "cpu")
    assert torch.equal(one["a.weight"], two["a.weight"])
    key = tensor_key(5, "a.weight")
    whole = host_values(key, "normal", 0.02, 0, 2000)
    np.testing.assert_array_equal(host_values(key, "normal", 0.02, 700, 100), whole[700:800])
    assert tensor_key(5, "a.weight") != tensor_key(5, "a.weighu") != tensor_key(6, "a.weight")
    # the shape of a normal distribution, not only its first two moments
    z = host_values(tensor_key(0, "shape"), "normal", 1.0, 0, 400000).astype(np.float64)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1) < 0.01
    assert abs((z ** 3).mean()) < 0.02 and abs((z ** 4).mean() - 3.0) < 0.06
    for x, p in ((-2.0, 0.02275), (-1.0, 0.158655), (0.0, 0.5), (0.5, 0.691462), (1.5, 0.933193), (3.0, 0.99865)):
        assert abs((z < x).mean() - p) < 0.003, x
    u = host_values(tensor_key(0, "u"), "around_one", 0.25, 0, 100000)
    assert 0.75 <= u.min() < 0.751 and 1.249 < u.max() < 1.25 and abs(u.mean() - 1) < 0.002
    ints = host_values(tensor_key(0, "i"), "int", 5, 0, 10000)
    assert ints.dtype == np.int32 and set(ints.tolist()) == {0, 1, 2, 3, 4}


def test_a_checkpoint_in_two_files_with_an_index(tmp_path):
    folder, cfg = make_folder(tmp_path, "B", "bfloat16")
    wanted = declared_tensors(cfg.model_spec())
    whole = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: whole.read(n).clone() for n in whole.names()}
    whole.close()
    (folder / "model.safetensors").unlink()
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[:len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fn, ns in shards.items():
        write_safetensors(folder / fn, {n: tensors[n] for n in ns})
    # without an index every *.safetensors file is opened
    got = bind_tensors(open_checkpoint(folder), wanted, torch.bfloat16, "cpu")
    assert all(torch.equal(got[n], tensors[n]) for n in names)
    # with an index only the files it names are opened: a stray file beside them does no harm
    index = {"metadata": {}, "weight_map": {n: fn for fn, ns in shards.items() for n in ns}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    write_safetensors(folder / "optimizer.safetensors", {"step": torch.zeros(1)})
    files = open_checkpoint(folder)
    assert [f.path.name for f in files] == sorted(shards)
    got = bind_tensors(files, wanted, torch.bfloat16, "cpu")
    assert all(torch.equal(got[n], tensors[n]) for n in names)
    # an index that points a tensor at the wrong file, or at a file that is not there
    bad = dict(index["weight_map"])
    bad[names[0]] = "model-00002-of-00002.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": bad}))
    with pytest.raises(qs.QStreamError, match=names[0].replace(".", r"\.")):
        open_checkpoint(folder)
    bad[names[0]] = "model-00003-of-00002.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": bad}))
    with pytest.raises(qs.QStreamError) as e:
        open_checkpoint(folder)
    assert e.value.code == qs.QsError.FILE_NOT_FOUND
    (folder / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(qs.QStreamError) as e:
        open_checkpoint(folder)
    assert e.value.code == qs.QsError.FILE_CORRUPTED


def test_fp32_matrices_in_a_bfloat16_engine(tmp_path, capsys):
    folder, cfg = make_folder(tmp_path, "A", "float32")
    wanted = declared_tensors(cfg.model_spec())
    kept = bind_tensors(open_checkpoint(folder), wanted, torch.bfloat16, "cpu")
    assert kept["lm_head.weight"].dtype == torch.float32
    assert "stored in 32-bit" in capsys.readouterr().err
    narrow = bind_tensors(open_checkpoint(folder), wanted, torch.bfloat16, "cpu", narrow_fp32_matrices=True)
    assert narrow["lm_head.weight"].dtype == torch.bfloat16
    assert torch.equal(narrow["lm_head.weight"], kept["lm_head.weight"].bfloat16())
    assert narrow["lm_head.bias"].dtype == narrow["transformer.ln_f.weight"].dtype == torch.float32
    assert "stored in 32-bit" not in capsys.readouterr().err


def test_mkmodel_writes_the_folder_that_the_library_writes(tmp_path):
    """`bin/qs-mkmodel` from a config.json and a seed: the same file as `write_model_folder`."""
    import subprocess
    import sys
    from pathlib import Path
    cfg_dict, scales, seed = TINY["A"]
    (tmp_path / "cfg.json").write_text(json.dumps({**cfg_dict, "architectures": ["GPTJForCausalLM"]}))
    tool = Path(__file__).resolve().parent.parent / "bin" / "qs-mkmodel"
    out = subprocess.run([sys.executable, str(tool), "--config", str(tmp_path / "cfg.json"), "--seed", str(seed),
                          "--out", str(tmp_path / "made"), "--dtype", "bfloat16", "--matrix-std", str(scales.matrix_std),
                          "--norm-spread", str(scales.norm_spread), "--bias-std", str(scales.bias_std)],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    folder, cfg = make_folder(tmp_path, "A", "bfloat16")
    assert (tmp_path / "made" / "model.safetensors").read_bytes() == (folder / "model.safetensors").read_bytes()
    assert json.loads((tmp_path / "made" / "config.json").read_text())["n_embd"] == 64
    bad = subprocess.run([sys.executable, str(tool), "--config", str(tmp_path / "nothing.json"), "--out", str(tmp_path / "x")],
                         capture_output=True, text=True)
    assert bad.returncode == 1 and "nothing.json" in bad.stderr
