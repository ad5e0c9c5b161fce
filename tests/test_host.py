"""CPU tests of the host side: validation contract, tritium rebinding, C-ABI loading, workload
generators and the bench harness's CPU arm. No kernel is launched here."""

from __future__ import annotations

import ctypes
import json
import subprocess
import sys
import types
from pathlib import Path

import pytest
import torch

import __graft_entry__ as entry
from helion_b200 import _lib, inputs, install, ops, parallel, uninstall

ROOT = Path(__file__).resolve().parent.parent


# ---- validation: same exceptions and messages as the reference ----------------------------------
def test_rejects_cpu_tensors():
    with pytest.raises(ValueError, match="hidden must be a CUDA tensor."):
        ops.linear_cross_entropy(torch.randn(4, 8), torch.randn(16, 8), torch.randint(16, (4,)))
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.linear_cross_entropy_backward(torch.tensor(1.0), torch.randn(4, 8), torch.randn(16, 8),
                                          torch.randint(16, (4,)), torch.randn(4))


@pytest.fixture()
def any_device(monkeypatch):
    """Lets the later checks be reached with CPU tensors (the first check is the device check)."""
    monkeypatch.setattr(ops, "_need_cuda", lambda name, t: None)


def _good():
    return torch.randn(4, 8), torch.randn(16, 8), torch.randint(16, (4,))


def test_validation_messages(any_device):
    h, w, t = _good()
    cases = [
        ((h.double(), w, t), "hidden must have one of these dtypes: float16, bfloat16, float32."),
        ((h, w.double(), t), "weight must have one of these dtypes"),
        ((h, w, t.float()), "target must have one of these dtypes: int32, int64."),
        ((h[0], w, t[0]), "hidden must have at least 2 dimensions"),
        ((h, w[0], t), "weight must be a 2D tensor shaped"),
        ((h, torch.randn(16, 9), t), "Shape mismatch: hidden has last dimension 8, weight expects 9."),
        ((h, w, torch.randint(16, (5,))), r"Shape mismatch: target has shape \(5,\), expected \(4,\)."),
        ((h, w.half(), t), "Dtype mismatch: weight has dtype torch.float16, hidden has dtype torch.float32."),
        ((h.t().contiguous().t(), w, t), "hidden must be contiguous for tritium.linear_cross_entropy."),
        ((h, w.t().contiguous().t(), t), "weight must be contiguous for tritium.linear_cross_entropy."),
    ]
    for args, msg in cases:
        with pytest.raises(ValueError, match=msg):
            ops.check_inputs(*args)
    with pytest.raises(ValueError, match="vocab_size must be positive."):
        ops.check_inputs(h, torch.randn(0, 8), t)
    assert ops.check_inputs(torch.randn(2, 3, 8), w, torch.randint(16, (2, 3))) == (6, 8, 16)


def test_validation_order_matches_reference(any_device):
    # dtype problems are reported before shape problems, shape before contiguity
    with pytest.raises(ValueError, match="dtypes"):
        ops.check_inputs(torch.randn(4).double(), torch.randn(16, 8), torch.randint(16, (4,)))
    with pytest.raises(ValueError, match="Shape mismatch"):
        ops.check_inputs(torch.randn(8, 4).t(), torch.randn(16, 9), torch.randint(16, (4,)))


def test_backward_validation_messages(any_device):
    h, w, t = _good()
    lse = torch.randn(4)
    bad = [
        ((torch.ones(1), h, lse, 4, ()), r"Shape mismatch: grad_out has shape \(1,\), expected \(\)."),
        ((torch.tensor(1.0), h, torch.randn(5), 4, ()), r"Shape mismatch: logsumexp has shape \(5,\), expected \(4,\)."),
        ((torch.tensor(1.0), h, lse.double(), 4, ()), "Dtype mismatch: logsumexp has dtype torch.float64, expected float32."),
        ((torch.tensor(1.0), h, torch.randn(8)[::2], 4, ()), "logsumexp must be contiguous"),
    ]
    for args, msg in bad:
        with pytest.raises(ValueError, match=msg):
            ops.check_backward_inputs(*args)


def test_plain_cross_entropy_validation_messages(any_device, monkeypatch):
    from helion_b200 import ce_ops

    monkeypatch.setattr(ce_ops, "_need_cuda", lambda name, t: None)
    z, t = torch.randn(4, 16), torch.randint(16, (4,))
    for args, msg in [
        ((z.double(), t), "logits must have one of these dtypes"),
        ((z[0], t), r"logits must be a 2D tensor shaped \(n_rows, vocab_size\)."),
        ((z, t[None]), "target must be a 1D tensor."),
        ((z, torch.randint(16, (5,))), r"Shape mismatch: target has shape \(5,\), expected \(4,\)."),
        ((torch.randn(16, 4).t(), t), "logits must be contiguous for tritium.cross_entropy."),
    ]:
        with pytest.raises(ValueError, match=msg):
            ce_ops.check_inputs(*args)
    assert ce_ops.check_inputs(torch.randn(3, 200000), torch.randint(9, (3,))) == (3, 200000)  # no vocabulary cap


def test_plain_cross_entropy_rejects_cpu_tensors():
    import helion_b200

    with pytest.raises(ValueError, match="CUDA tensor"):  # the reference's own test (test_cross_entropy.py:112-114)
        helion_b200.cross_entropy(torch.randn(4, 16), torch.randint(16, (4,)))


def test_unknown_reduction_is_rejected(any_device):
    with pytest.raises(ValueError, match="reduction must be one of"):
        ops._check_reduction("batchmean")


# ---- install(): rebinding the reference's module attributes ---------------------------------------
def _fake_tritium():
    root = types.ModuleType("fake_tritium")
    sub = types.ModuleType("fake_tritium.ops")
    leaf = types.ModuleType("fake_tritium.ops.cross_entropy")
    for mod in (root, sub, leaf):
        mod.linear_cross_entropy = lambda *a: "reference forward"
        mod.linear_cross_entropy_backward = lambda *a: "reference backward"
        mod.cross_entropy = lambda *a: "reference plain forward"
        mod.cross_entropy_backward = lambda *a: "reference plain backward"
        mod.layernorm = lambda *a: "another op"
    root.ops = sub
    # on tritium.ops the attribute `cross_entropy` is the function (it shadows the submodule)
    for mod in (root, sub, leaf):
        sys.modules[mod.__name__] = mod
    return root, sub, leaf


def test_install_rebinds_all_three_modules_and_uninstall_restores():
    from helion_b200 import ce_ops

    root, sub, leaf = _fake_tritium()
    try:
        rebound = install(root)
        assert len(rebound) == 12  # (the fake package has no matmul module)
        for mod in (root, sub, leaf):
            assert mod.linear_cross_entropy is ops.linear_cross_entropy
            assert mod.linear_cross_entropy_backward is ops.linear_cross_entropy_backward
            assert mod.cross_entropy is ce_ops.cross_entropy
            assert mod.cross_entropy_backward is ce_ops.cross_entropy_backward
            assert mod.layernorm() == "another op"  # everything else is left alone
        install(root)  # idempotent: the saved originals are not overwritten by our own functions
        uninstall(root)
        for mod in (root, sub, leaf):
            assert mod.linear_cross_entropy() == "reference forward"
            assert mod.linear_cross_entropy_backward() == "reference backward"
            assert mod.cross_entropy() == "reference plain forward"
    finally:
        for name in list(sys.modules):
            if name.startswith("fake_tritium"):
                del sys.modules[name]


def test_install_into_the_real_reference_package_if_present():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "tritium").exists():
        pytest.skip("reference not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        import tritium

        original = tritium.linear_cross_entropy
        install()
        assert tritium.linear_cross_entropy is ops.linear_cross_entropy
        assert sys.modules["tritium.ops.cross_entropy"].linear_cross_entropy_backward is ops.linear_cross_entropy_backward
        from helion_b200 import norm_ops

        assert tritium.residual_rmsnorm is norm_ops.residual_rmsnorm
        assert sys.modules["tritium.ops.rmsnorm"].rmsnorm_backward is norm_ops.rmsnorm_backward
        with pytest.raises(ValueError, match="CUDA tensor"):
            tritium.linear_cross_entropy(torch.randn(4, 8), torch.randn(16, 8), torch.randint(16, (4,)))
        uninstall()
        assert tritium.linear_cross_entropy is original
    finally:
        sys.path.remove(str(ref))


# ---- the C ABI -------------------------------------------------------------------------------------
def test_library_loads_and_exports_every_declared_symbol():
    handle = _lib.lib()
    declared = entry.declared_symbols()
    assert "lce_forward_stats" in declared and "lce_backward" in declared and len(declared) >= 11
    for name in declared:
        assert hasattr(handle, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert handle.lce_version() == 2
    assert handle.lce_strerror(0) == b"ok"
    assert b"workspace" in handle.lce_strerror(3)
    assert isinstance(handle.lce_launch_count(), int)


def test_workspace_sizing_is_host_only_and_sane():
    L = _lib.lib()
    bf16 = _lib.DTYPE_BF16
    # forward: 3 floats per (vocab tile, row)
    tc = L.lce_forward_workspace_bytes(8192, 4096, 128256, bf16, _lib.FLAG_FORCE_TC)
    assert 501 * 3 * 8192 * 4 <= tc <= 501 * 3 * 8192 * 4 + 4096
    assert L.lce_forward_workspace_bytes(8192, 4096, 128256, bf16, 0) >= tc
    assert L.lce_forward_workspace_bytes(-1, 4096, 10, bf16, 0) == 0
    assert L.lce_finalize_workspace_bytes(1000) >= 4000
    # backward: never an N x V buffer; the G block obeys the byte cap
    n, h, v = 8192, 4096, 128256
    full_logits = n * v * 2
    default = L.lce_backward_workspace_bytes(n, h, v, bf16, 0, 0)
    assert default < full_logits // 3
    # a tighter cap shrinks the G block; what it adds is fp32 partial-sum scratch of dX / dW size
    small = L.lce_backward_workspace_bytes(n, h, v, bf16, 0, 64 << 20)
    assert 0 < small <= (64 << 20) + 4 * (n * h + v * h) * 2
    # one block covers everything when it fits; the only extra is the split-K slabs of the dX GEMM
    # (a few 128 x 256 fp32 tiles) that let a problem with this few rows fill the GPU
    tiny = L.lce_backward_workspace_bytes(128, 64, 1024, bf16, 0, 0)
    assert tiny < 128 * 1024 * 2 + 16 * 2 * 128 * 256 * 4 + 8192


def test_null_pointers_and_bad_enums_are_argument_errors():
    L = _lib.lib()
    assert L.lce_forward_stats(None, None, None, 1, 8, 8, 8, 0, 0, None, None, 0, 0, None) == 1
    assert L.lce_forward_stats(None, None, None, 1, 8, 8, 8, 0, 7, None, None, 0, 0, None) == 1
    assert L.lce_backward(None, None, None, 1, None, None, 8, 8, 8, 0, 0, -100, 9, None, None, None, 0, 0, 0, None, None, None, None) == 1
    plan = (ctypes.c_int64 * 4)()
    assert L.lce_backward_plan(8192, 4096, 128256, 0, 0, 0, None, None, plan) == 0
    assert list(plan) == [8192, 16384, 1, 8]  # Llama-3 head: all rows, 8 vocabulary bands of 16384 columns
    assert L.lce_backward_plan(65536, 5120, 19008, 0, 0, 0, None, None, plan) == 0
    assert plan[2] > 1 and plan[0] * plan[1] * 2 <= 256 << 20  # 14B-class shard: row chunks, block under the cap
    with pytest.raises(_lib.LceError, match="invalid argument"):
        _lib.check(1, "lce_forward_stats")


def test_ops_fail_loudly_without_the_library(monkeypatch):
    _lib.lib.cache_clear()
    monkeypatch.setattr(_lib._build, "build_library", lambda *a, **k: (_ for _ in ()).throw(RuntimeError("no nvcc")))
    try:
        with pytest.raises(RuntimeError, match="no fallback"):
            _lib.lib()
    finally:
        _lib.lib.cache_clear()


# ---- workloads -------------------------------------------------------------------------------------
def test_config_generators_are_seeded_and_shaped():
    cfg = inputs.scaled(inputs.CONFIGS["llama3-8b"], rows=512, hidden=64, vocab=2000)
    a, b = inputs.make_inputs(cfg), inputs.make_inputs(cfg)
    for key in ("hidden", "weight", "target"):
        assert torch.equal(a[key], b[key])
    assert a["hidden"].shape == (1, 512, 64) and a["hidden"].dtype == torch.bfloat16
    assert a["weight"].shape == (2000, 64) and a["target"].dtype == torch.int64
    assert int((a["target"] == -100).sum()) == round(0.02 * 512)
    rms = a["hidden"].float().pow(2).mean(dim=-1).sqrt()
    assert torch.allclose(rms, torch.ones_like(rms), atol=2e-2)
    assert abs(float(a["weight"].float().std()) - 0.02) < 2e-3
    live = a["target"][a["target"] >= 0]
    assert 0 <= int(live.min()) and int(live.max()) < 2000
    # Zipf: the most frequent token is far above the uniform rate
    assert int(torch.bincount(live).max()) > 5 * 512 / 2000


def test_named_configs_have_the_benchmark_shapes():
    c = inputs.CONFIGS
    assert (c["gpt2-small"].rows, c["gpt2-small"].hidden, c["gpt2-small"].vocab) == (4096, 768, 50304)
    assert (c["llama3-8b"].rows, c["llama3-8b"].hidden, c["llama3-8b"].vocab) == (8192, 4096, 128256)
    assert (c["large-vocab"].rows, c["large-vocab"].hidden, c["large-vocab"].vocab) == (16384, 2304, 256000)
    assert (c["14b-class"].rows, c["14b-class"].hidden, c["14b-class"].vocab) == (65536, 5120, 152064)
    assert c["14b-class"].reduction == "sum" and c["14b-class"].grad_out == 1 / 65536
    assert inputs.sweep_config(1024).rows == 1024


def test_shard_bounds_partition_the_vocabulary():
    for vocab, world in [(128256, 8), (1003, 4), (7, 8)]:
        spans = [parallel.shard_bounds(vocab, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == vocab
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert parallel.shard_bounds(128256, 8, 3) == (3 * 16032, 4 * 16032)


# ---- bench.py: the CPU (reference) arm runs without a GPU ----------------------------------------
def test_bench_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "smoke",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["higher_is_better"] is True
    assert line["config"]["workload"] == "smoke"


def test_greedy_head_rejects_cpu_tensors_before_touching_the_library():
    from helion_b200 import decode_ops

    with pytest.raises(ValueError, match="hidden must be a CUDA tensor"):
        decode_ops.greedy_head(torch.randn(2, 8), torch.randn(16, 8))


def test_oracle_greedy_expression_is_argmax_of_log_softmax():
    from oracle import oracle

    g = torch.Generator().manual_seed(3)
    h, w = torch.randn(2, 5, 16, generator=g).bfloat16(), torch.randn(40, 16, generator=g).bfloat16()
    e = oracle.greedy_expression(h, w)
    ls = torch.log_softmax(h.float().reshape(-1, 16) @ w.float().T, dim=-1)
    assert torch.equal(e["token"].reshape(-1), ls.argmax(dim=-1))
    torch.testing.assert_close(e["logprob"].reshape(-1), ls.max(dim=-1).values, rtol=1e-6, atol=1e-6)


def test_grad_norm_hand_over_matches_only_the_untouched_gradient():
    """The registry that hands the dW epilogue's sum of squares to grad_sumsq: a hit needs the same storage,
    address, shape and version; a clone, a written tensor or a freed one miss; autograd's hand-over of a leaf
    gradient (no copy) hits."""
    from helion_b200 import grad_norm

    grad_norm.enable(True)
    try:
        g, s = torch.randn(5, 3), torch.tensor(1.0)
        grad_norm.remember(g, s)
        assert grad_norm.lookup(g) is s
        assert grad_norm.lookup(g.clone()) is None and grad_norm.lookup(g[:2]) is None
        g.mul_(2.0)
        assert grad_norm.lookup(g) is None

        class Op(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x):
                return x.sum()

            @staticmethod
            def backward(ctx, go):
                dw = torch.full((4,), 2.0) * go
                grad_norm.remember(dw, torch.tensor(16.0))
                return dw

        x = torch.zeros(4, requires_grad=True)
        Op.apply(x).backward()
        assert float(grad_norm.lookup(x.grad)) == 16.0
        Op.apply(x).backward()  # accumulates into the existing .grad: the remembered sum no longer applies
        assert grad_norm.lookup(x.grad) is None
        for _ in range(3 * grad_norm.KEEP):
            grad_norm.remember(torch.randn(2), s)
        assert len(grad_norm._known) <= grad_norm.KEEP
    finally:
        grad_norm.enable(False)
    assert not grad_norm._known
