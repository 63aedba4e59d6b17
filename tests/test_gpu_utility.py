"""The utility kernels: seeded random fill (host twin bit for bit), conversion at upload, the finite
check, canary words, token feed and page clearing."""
import numpy as np
import pytest
import torch

import qstream_b200 as qs
from qstream_b200.csrc import ops
from qstream_b200.engine.model import declared_tensors
from qstream_b200.weights.random_init import host_values, random_tensors, tensor_key
from util import TINY

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,a", [("normal", 0.02), ("normal", 1.0), ("around_one", 0.1)])
def test_random_fill_is_the_same_on_host_and_device(dtype, kind, a):
    n = 1 << 20
    key = tensor_key(7, f"transformer.h.3.mlp.fc_in.weight/{kind}")
    dev = ops.random_fill(torch.empty(n, dtype=dtype, device="cuda"), key, {"normal": 0, "around_one": 1}[kind], a)
    host = torch.from_numpy(host_values(key, kind, a, 0, n)).to(dtype)
    assert torch.equal(dev.cpu(), host)
    # a slice far into a large tensor is the stream's own elements there
    first = 5_000_000_123
    dev = ops.random_fill(torch.empty(4096, dtype=dtype, device="cuda"), key, {"normal": 0, "around_one": 1}[kind], a, first)
    assert torch.equal(dev.cpu(), torch.from_numpy(host_values(key, kind, a, first, 4096)).to(dtype))


def test_random_fill_integers_and_refusals():
    key = tensor_key(1, "table")
    dev = ops.random_fill(torch.empty(10000, dtype=torch.int32, device="cuda"), key, 2, 7)
    assert torch.equal(dev.cpu(), torch.from_numpy(host_values(key, "int", 7, 0, 10000)))
    assert 0 <= int(dev.min()) and int(dev.max()) == 6
    with pytest.raises(qs.QStreamError):
        ops.random_fill(torch.empty(8, dtype=torch.float32, device="cuda"), key, 2, 7)        # integers into floats
    with pytest.raises(qs.QStreamError):
        ops.random_fill(torch.empty(8, dtype=torch.float16, device="cuda"), key, 0, 1.0)


@pytest.mark.parametrize("which", ["A", "B"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_model_made_on_the_device_is_the_folder_the_host_writes(which, dtype):
    cfg_dict, scales, seed = TINY[which]
    cfg = qs.GptjConfig.from_dict({**cfg_dict, "architectures": ["GPTJForCausalLM"]})
    wanted = declared_tensors(cfg.model_spec())
    host = random_tensors(wanted, seed, dtype, "cpu", scales)
    dev = random_tensors(wanted, seed, dtype, "cuda", scales)
    assert host.keys() == dev.keys()
    for name in host:
        assert torch.equal(host[name], dev[name].cpu()), name
    other = random_tensors(wanted, seed + 1, dtype, "cuda", scales)
    assert not torch.equal(other["lm_head.weight"], dev["lm_head.weight"])


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float16, torch.float32), (torch.float16, torch.bfloat16),
                                     (torch.float32, torch.float32)])
def test_convert(src, dst):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(100003, generator=g) * 10).to(src)
    x[:6] = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 6e-8, 65504.0]).to(src)
    got = ops.convert(x.cuda(), dst)
    assert got.dtype == dst and torch.equal(got.cpu(), x.to(dst))
    nan = ops.convert(torch.tensor([float("nan")], dtype=src).cuda(), dst)
    assert torch.isnan(nan).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_check_finite(dtype):
    x = torch.randn(37, 130).to(dtype).cuda()
    wide = torch.zeros(37, 200, dtype=dtype).cuda()
    wide[:, :130] = x
    record = torch.zeros(4, dtype=torch.int32).cuda()
    ops.check_finite(wide[:, :130], 5, record)
    assert record.tolist() == [0, 0, 0, 0]
    wide[:, 130:] = float("nan")                       # beyond the rows' width: not scanned
    ops.check_finite(wide[:, :130], 5, record)
    assert record.tolist() == [0, 0, 0, 0]
    wide[20, 77] = float("inf")
    slots = torch.zeros(37, dtype=torch.int32).cuda()
    slots[20] = -1
    ops.check_finite(wide[:, :130], 6, record, slots)  # a padding row is skipped
    assert record.tolist() == [0, 0, 0, 0]
    ops.check_finite(wide[:, :130], 7, record)
    assert record.tolist() == [1, 7, 20, 77]
    wide[3, 0] = float("nan")
    ops.check_finite(wide[:, :130], 8, record)         # the first report stays
    assert record.tolist() == [1, 7, 20, 77]


def test_canary_words():
    buf = torch.zeros(1000, dtype=torch.int32).cuda()
    damaged = torch.zeros(2, dtype=torch.int32).cuda()
    ops.canary_fill(buf, 0xC0FFEE11)
    ops.canary_check(buf, 0xC0FFEE11, damaged)
    assert damaged.tolist() == [0, 0]
    buf[613] += 1
    ops.canary_check(buf, 0xC0FFEE11, damaged)
    assert damaged.tolist() == [1, 613]


def test_take_tokens_and_zero_pages():
    dst = torch.full((8,), 7, dtype=torch.int32).cuda()
    src = torch.tensor([10, 11, 12], dtype=torch.int32).cuda()
    idx = torch.tensor([2, -1, 0, 5, 1, 0, 0, 0], dtype=torch.int32).cuda()
    ops.take_tokens(dst, src, idx, 5)
    assert dst.tolist() == [12, 7, 10, 7, 11, 7, 7, 7]             # -1 and an index outside keep the host's token
    store = torch.ones(3, 5, 2, 64, 16, dtype=torch.bfloat16).cuda()
    ops.zero_pages(store, torch.tensor([4, 1], dtype=torch.int32).cuda())
    assert (store[:, [1, 4]] == 0).all() and (store[:, [0, 2, 3]] == 1).all()


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable(tmp_path):
    """The library's bounded wait on a barrier that nothing completes: it gives up after its polls, the kernel
    records a status code and returns; the host reads the code through the engine's `check_status`, and the
    next step runs as if nothing had happened.  (No kernel of the model is made to fail for this.)"""
    from util import make_folder
    status = torch.zeros(1, dtype=torch.int32).cuda()
    ops.selftest_bounded_wait(status, polls=500)
    torch.cuda.synchronize()
    assert int(status.item()) == 199
    folder, cfg = make_folder(tmp_path, "A", "bfloat16")
    eng = qs.Engine(qs.load_model(folder, dtype="bfloat16", device="cuda"), max_tokens=128, max_batch=1)
    slot = eng.acquire()
    first = eng.step([slot], [[1, 2, 3]]).clone()
    eng.check_status()
    ops.selftest_bounded_wait(eng.status, polls=500)
    with pytest.raises(qs.QStreamError) as e:
        eng.check_status()
    assert e.value.code == qs.QsError.INTERNAL and "ran out" in str(e.value)
    eng.release(slot)
    slot = eng.acquire()
    assert torch.equal(eng.step([slot], [[1, 2, 3]]), first)
    eng.check_status()
