"""CPU: host-side logic of the python mirrors (no kernels run)."""
import numpy as np
import pytest
import torch

from qtip_b200 import kernel_check, ops, qtip_kernels
from qtip_b200.quantized_linear import QuantizedLinear


def test_pack_hadk_round_trip():
    for k in (12, 28, 52, 172):
        h = ops.get_hadK(k * 4)[0]
        bits = ops.pack_hadk(h).numpy().view(np.uint32)
        assert bits.shape == (k, (k + 31) // 32)
        un = ((bits[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(k, -1)[:, :k]
        assert np.array_equal(un.astype(np.float32) * 2 - 1, h.numpy())


def test_get_hadk_contract():
    assert ops.get_hadK(4096) == (None, 1)
    h, k = ops.get_hadK(11008)
    assert k == 172 and h.shape == (172, 172) and h.dtype == torch.float32
    ht, _ = ops.get_hadK(11008, transpose=True)
    assert torch.equal(ht, h.T)
    with pytest.raises(ValueError):
        ops.get_hadK(172 * 3)


def test_has_kernel_predicate():
    assert kernel_check.has_kernel('quantlut_sym', 16, 2, 2, 9, 16, 16)
    assert not kernel_check.has_kernel('3inst', 16, 2, 1, 0, 16, 16)
    assert not kernel_check.has_kernel('quantlut_sym', 16, 5, 2, 9, 16, 16)
    assert not kernel_check.has_kernel('quantlut_sym', 16, 2, 2, 8, 16, 16)


def test_legacy_kernel_names_resolve():
    f = qtip_kernels.decompress_matvec_16_9_2_1_4096_1_11008
    assert callable(f) and f is qtip_kernels.decompress_matvec_16_9_2_1_4096_1_11008
    with pytest.raises(AttributeError):
        qtip_kernels.decompress_matvec_16_9_5_1_4096_1_4096
    with pytest.raises(AttributeError):
        qtip_kernels.decompress_matvec_16_8_2_1_4096_1_4096
    with pytest.raises(AttributeError):
        qtip_kernels.something_else
    with pytest.raises(RuntimeError, match="CUDA"):
        f(torch.zeros(4096, 1), torch.zeros(8, dtype=torch.int32), torch.zeros(11008, 1, dtype=torch.float16),
          torch.zeros(1024, dtype=torch.float16))


def test_upstream_codebook_package_imports_on_the_shim():
    """lib/codebook/__init__.py upstream, unmodified, registers its 61 quip_lib ops against this package installed as
    `qtip_kernels`, and every kernel name it calls resolves (needs a checkout: QTIP_REFERENCE_ROOT)."""
    import os
    import subprocess
    import sys
    root = os.environ.get("QTIP_REFERENCE_ROOT")
    if not root or not os.path.isdir(os.path.join(root, "lib", "codebook")):
        pytest.skip("QTIP_REFERENCE_ROOT is not set to an upstream checkout")
    code = (
        "import sys, torch\n"
        "import qtip_b200; qtip_b200.install_as_qtip_kernels()\n"
        f"sys.path.insert(0, {root!r})\n"
        "import lib.codebook as cb, qtip_kernels\n"
        "assert len(cb.kernels) == 61\n"
        "for m, n, k, r in cb.kernels:\n"
        "    assert callable(getattr(qtip_kernels, f'decompress_matvec_16_9_{r}_1_{m}_{n}_{k}'))\n"
        "    op = getattr(torch.ops.quip_lib, f'decompress_matvec_qtip_{m}_{n}_{k}_{r}')\n"
        "from torch._subclasses.fake_tensor import FakeTensorMode\n"
        "with FakeTensorMode():\n"
        "    y = torch.ops.quip_lib.decompress_matvec_qtip_4096_1_4096_2(torch.zeros(65536, 32, dtype=torch.int16),\n"
        "        torch.zeros(1, 4096, dtype=torch.float16), torch.zeros(512, 2, dtype=torch.float16))\n"
        "    assert tuple(y.shape) == (1, 4096)\n"
        "print('shim ok')\n")
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=here, timeout=300)
    assert r.returncode == 0 and "shim ok" in r.stdout, r.stderr[-2000:]


def test_quantized_linear_state_dict_keys():
    q = QuantizedLinear(11008, 4096, 16, 16, 16, 2, 2, 9, 'quantlut_sym')
    sd = q.state_dict()
    assert set(sd) == {"rcp", "tp_rank", "trellis", "tlut", "SU", "SV"}
    assert sd["trellis"].shape == (4096 // 16 * 11008 // 16, 32) and sd["trellis"].dtype == torch.int16
    assert sd["tlut"].shape == (512, 2) and sd["tlut"].dtype == torch.float16
    assert sd["SU"].dtype == torch.float16 and sd["SV"].dtype == torch.float32
    assert q.K_left == 172 and q.K_right == 1 and q.has_kernel
    q3 = QuantizedLinear(256, 256, 16, 16, 16, 2, 1, 0, '3inst')
    assert q3.tlut is None and not q3.has_kernel


def test_unpack_quip_scale_folding():
    """lib/utils/data_utils.py:281-307 upstream: where the weight scale goes for rcp 0 / 1 / 2."""
    from qtip_b200.checkpoint import unpack_quip
    m, n, K = 64, 128, 2
    g = torch.Generator().manual_seed(0)
    base = dict(trellis=torch.randint(-2**15, 2**15, (m * n // 256, 16 * K), generator=g).to(torch.int16),
                SU=torch.randn(n, generator=g).sign().half(), SV=torch.randn(m, generator=g).sign().half(),
                tlut=torch.randn(512, 2, generator=g).half())
    q = unpack_quip(QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, 'quantlut_sym'), dict(base, Wscale=torch.tensor(0.5)))
    assert torch.equal(q.SV, base["SV"].float() * 0.5) and torch.equal(q.SU, base["SU"]) and int(q.rcp) == 0
    assert torch.equal(q.trellis, base["trellis"]) and torch.equal(q.tlut.data, base["tlut"])
    ws = torch.arange(1, 9).float()
    q = unpack_quip(QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, 'quantlut_sym'), dict(base, Wscale=ws, rcp=1, tp_rank=8))
    assert int(q.rcp) == 1 and int(q.tp_rank) == 8 and torch.equal(q.SV, base["SV"].float())
    assert torch.equal(q.SU.float(), (base["SU"].float().reshape(8, -1) * ws[:, None]).reshape(-1))
    q = unpack_quip(QuantizedLinear(n, m, 16, 16, 16, K, 2, 9, 'quantlut_sym'), dict(base, Wscale=ws, rcp=2, tp_rank=8))
    assert int(q.rcp) == 2 and torch.equal(q.SU, base["SU"])
    assert torch.equal(q.SV, (base["SV"].float().reshape(8, -1) * ws[:, None]).reshape(-1))


def test_torch_ops_register_with_fake_impl():
    from qtip_b200 import codebook_ops
    assert len(codebook_ops.UPSTREAM_TABLE) == 61
    op = codebook_ops.register(4096, 11008, 2)
    assert op is codebook_ops.register(4096, 11008, 2)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        y = op(torch.empty(4096 * 11008 // 256, 32, dtype=torch.int16), torch.empty(1, 11008), torch.empty(512, 2, dtype=torch.float16))
        assert y.shape == (1, 4096) and y.dtype == torch.float32


def test_wrappers_refuse_tensors_of_another_device(monkeypatch):
    """The preallocated-tensor wrappers launch on the current device: a tensor that lives on another GPU must be
    refused on the host, before any launch (no GPU needed: the device query is faked)."""
    import types
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 1)
    on0 = types.SimpleNamespace(device=types.SimpleNamespace(index=0))
    on1 = types.SimpleNamespace(device=types.SimpleNamespace(index=1))
    ops._check_device(on1, None, on1)
    with pytest.raises(RuntimeError, match="current device"):
        ops._check_device(on1, on0)
    for fn, args in ((ops.embed_token, (on0, on0, on0, on0)), (ops.lm_head, (on0, on0, on0, on0, types.SimpleNamespace(
            device=on0.device, shape=(8, 8)), 1e-5)), (ops.attn_decode, (on0, on0, on0, on0, on0, 1, 1, 128)),
                     (ops.rope_kv_append, (on0, on0, on0, on0, on0, on0, 1, 1, 128))):
        with pytest.raises(RuntimeError, match="current device"):
            fn(*args)


def test_decode_model_refuses_more_positions_than_the_cache_holds():
    """QtipLlama.feed / generate count positions on the host and raise before a step would index past the caches."""
    from qtip_b200.llama import QtipLlama
    m = QtipLlama.__new__(QtipLlama)          # host bookkeeping only: no device buffers
    m.max_positions, m.steps_done = 10, 0
    m._reserve(6)
    m._reserve(4)
    with pytest.raises(RuntimeError, match="KV cache holds 10"):
        m._reserve(1)
    assert m.steps_done == 10


def test_quip_params_validation():
    """The config dict upstream stores in the HF config: what the decode path builds is accepted, everything else is
    refused with the key named (quantize_llama/quantize_finetune_llama.py:116-129, model/llama.py:306-317, 445-452)."""
    from qtip_b200.checkpoint import check_quip_params
    from qtip_b200.llama import LlamaShape
    shape = LlamaShape(K=2)
    ok = dict(codebook="bitshift", codebook_version=0, L=16, K=2, V=2, tlut_bits=9, decode_mode="quantlut_sym", td_x=16,
              td_y=16, split_for_tp=False, skip_list=None)
    assert check_quip_params(ok, shape) == 2
    for key, bad in (("L", 12), ("V", 1), ("tlut_bits", 8), ("decode_mode", "3inst"), ("td_x", 8), ("K", 5)):
        with pytest.raises(ValueError, match=key):
            check_quip_params(dict(ok, **{key: bad}), shape)
    with pytest.raises(ValueError, match="K_v_proj"):
        check_quip_params(dict(ok, K_v_proj=3), shape)
    with pytest.raises(ValueError, match="skip_list"):
        check_quip_params(dict(ok, skip_list=["0_q"]), shape)
    with pytest.raises(ValueError, match="built for K"):
        check_quip_params(dict(ok, K=3), shape)


def test_bench_arms_print_the_same_config():
    """Both arms of bench.py derive `config` from the same rule: fused q||k||v / gate||up matrices for the 7B shape on one
    GPU at batch 1, separate matrices everywhere else."""
    import argparse
    import importlib.util
    import os
    from conftest import ROOT
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    base = dict(separate_qkv=False, workload="llama2-7b", gpus=1, batch=1, prompt=128)
    ns = argparse.Namespace(**base)
    os.environ.pop("WORLD_SIZE", None)
    assert bench.use_fused_matrices(ns)
    assert "fused_matrices" in bench.workload_config(ns.workload, ns.prompt, 1, bench.use_fused_matrices(ns))
    for change in (dict(separate_qkv=True), dict(workload="llama3-405b"), dict(gpus=2), dict(batch=8)):
        assert not bench.use_fused_matrices(argparse.Namespace(**dict(base, **change))), change
    assert "fused_matrices" not in bench.workload_config("llama3-405b", 256, 8, False)
    assert bench.algorithmic_bytes(4096, 4096, 2) == 4210688
