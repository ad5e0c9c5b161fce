"""Parity of the sm_100a kernels with the oracle, through the public op and the C ABI. GPU only."""

from __future__ import annotations

import importlib.util
import math
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from _helpers import FP32_TOL, GRAD_RTOL_16BIT, LOSS_RTOL, reference_tolerances, rel_loss_err, scaled_max_err
from helion_b200 import _lib, inputs, install, ops, uninstall
from oracle import oracle

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_env_and_status(monkeypatch):
    monkeypatch.delenv("HELION_B200_FORCE", raising=False)
    monkeypatch.delenv("HELION_B200_BLOCK_BYTES", raising=False)
    yield
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a kernel reported a bounded wait that ran out"


def _run(x, w, t, *, reduction="mean", grad_out=None, ignore_index=-100):
    xd = x.to(DEV).requires_grad_(True)
    wd = w.to(DEV).requires_grad_(True)
    loss = ops.linear_cross_entropy(xd, wd, t.to(DEV), reduction=reduction, ignore_index=ignore_index)
    if grad_out is None:
        grad_out = torch.ones_like(loss)
    loss.backward(grad_out.to(DEV))
    torch.cuda.synchronize()
    return loss, xd.grad, wd.grad


def _check(x, w, t, *, reduction="mean", grad_out=None, ignore_index=-100):
    ref = oracle.expression(x, w, t, reduction=reduction, grad_out=grad_out, ignore_index=ignore_index)
    loss, dx, dw = _run(x, w, t, reduction=reduction, grad_out=grad_out, ignore_index=ignore_index)
    assert loss.dtype == torch.float32 and dx.dtype == x.dtype and dw.dtype == w.dtype
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    tol = FP32_TOL * 10 if x.dtype == torch.float32 else GRAD_RTOL_16BIT
    assert scaled_max_err(dx.reshape(ref["dx"].shape), ref["dx"]) <= tol
    assert scaled_max_err(dw, ref["dw"]) <= tol
    return loss, dx, dw


# ---- the reference's own tests, restated (tests/tritium/test_cross_entropy.py:59-122) --------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab_size", [128, 1024])
@pytest.mark.parametrize("n_rows", [1, 16, 128])
def test_linear_cross_entropy_forward(dtype, vocab_size, n_rows):
    hidden = torch.randn(n_rows, 64, device=DEV, dtype=dtype)
    weight = torch.randn(vocab_size, 64, device=DEV, dtype=dtype)
    target = torch.randint(vocab_size, (n_rows,), device=DEV)
    loss = ops.linear_cross_entropy(hidden, weight, target)
    ref = F.cross_entropy(F.linear(hidden, weight).float(), target)
    torch.testing.assert_close(loss, ref, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_cross_entropy_autograd(dtype):
    hidden = torch.randn(32, 64, device=DEV, dtype=dtype, requires_grad=True)
    weight = torch.randn(256, 64, device=DEV, dtype=dtype, requires_grad=True)
    target = torch.randint(256, (32,), device=DEV)
    ops.linear_cross_entropy(hidden, weight, target).backward()
    hidden_ref = hidden.detach().float().clone().requires_grad_(True)
    weight_ref = weight.detach().float().clone().requires_grad_(True)
    F.cross_entropy(F.linear(hidden_ref, weight_ref), target).backward()
    rtol, atol = reference_tolerances(dtype)
    torch.testing.assert_close(hidden.grad, hidden_ref.grad.to(dtype), rtol=rtol, atol=atol)
    rtol, atol = reference_tolerances(dtype, accumulated=True)
    torch.testing.assert_close(weight.grad, weight_ref.grad.to(dtype), rtol=rtol, atol=atol)


def test_linear_cross_entropy_accepts_3d_hidden():
    hidden = torch.randn(4, 16, 64, device=DEV, dtype=torch.float32)
    weight = torch.randn(128, 64, device=DEV, dtype=torch.float32)
    target = torch.randint(128, (4, 16), device=DEV)
    loss = ops.linear_cross_entropy(hidden, weight, target)
    ref = F.cross_entropy(F.linear(hidden, weight).view(-1, 128), target.view(-1))
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-4)


def test_rejects_non_contiguous_and_mixed_devices():
    hidden = torch.randn(64, 16, device=DEV).T
    with pytest.raises(ValueError, match="contiguous"):
        ops.linear_cross_entropy(hidden, torch.randn(8, 64, device=DEV), torch.randint(8, (16,), device=DEV))
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.linear_cross_entropy(torch.randn(16, 64, device=DEV), torch.randn(8, 64), torch.randint(8, (16,), device=DEV))


def test_drop_in_through_the_installed_reference_package():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "tritium").exists():
        pytest.skip("reference not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        import tritium

        install()
        hidden = torch.randn(4, 16, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        weight = torch.randn(300, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        target = torch.randint(300, (4, 16), device=DEV)
        before = _lib.lib().lce_launch_count()
        loss = tritium.linear_cross_entropy(hidden, weight, target)
        loss.backward()
        assert _lib.lib().lce_launch_count() > before  # our kernels ran, not the reference's
        ref_loss = F.cross_entropy(F.linear(hidden, weight).float().view(-1, 300), target.view(-1))
        torch.testing.assert_close(loss, ref_loss, rtol=2e-2, atol=2e-3)
        lse = torch.logsumexp(F.linear(hidden, weight).float().view(-1, 300), dim=-1)
        dx, dw = tritium.linear_cross_entropy_backward(torch.tensor(1.0, device=DEV), hidden.detach(), weight.detach(),
                                                       target, lse)
        assert dx.shape == (64, 64) and dw.shape == (300, 64)
        torch.testing.assert_close(dx.view(4, 16, 64), hidden.grad, rtol=2e-2, atol=2e-2)
    finally:
        uninstall()
        sys.path.remove(str(ref))


# ---- golden fixtures -------------------------------------------------------------------------------
CASES = make_golden.case_list()  # the plain-op cases at the end are covered by test_gpu_plain_ce.py
LINEAR_CASE_COUNT = sum(1 for c in CASES if c.get("op") != "plain")
ORACLE_FIXTURE = torch.load(GOLDEN / "oracle_cases.pt", weights_only=False)
REFERENCE_FIXTURE = torch.load(GOLDEN / "reference_b200.pt", weights_only=False)


@pytest.mark.parametrize("index", range(LINEAR_CASE_COUNT), ids=[c["name"] for c in CASES[:LINEAR_CASE_COUNT]])
def test_against_committed_fixtures(index):
    case = CASES[index]
    inp = make_golden.make_case_inputs(case, index)
    exp = ORACLE_FIXTURE[case["name"]]["expected"]
    ref = REFERENCE_FIXTURE[case["name"]]
    dtype = inp["hidden"].dtype
    xd = inp["hidden"].to(DEV).requires_grad_(case["grads"])
    wd = inp["weight"].to(DEV).requires_grad_(case["grads"])
    loss = ops.linear_cross_entropy(xd, wd, inp["target"].to(DEV))
    assert rel_loss_err(loss, exp["loss"]) <= LOSS_RTOL
    torch.testing.assert_close(loss.cpu(), ref["loss"], rtol=2e-2, atol=2e-3)  # vs the reference's kernels
    if case["grads"]:
        loss.backward(inp["grad_out"].to(DEV))
        tol = FP32_TOL * 10 if dtype == torch.float32 else GRAD_RTOL_16BIT
        assert scaled_max_err(xd.grad, exp["dx"].reshape(xd.shape)) <= tol
        assert scaled_max_err(wd.grad, exp["dw"]) <= tol
        if not case["name"].startswith("chunkloop") or dtype == torch.float32:
            # (the reference's 16-bit chunk loop rounds its logits; it is several percent off the truth)
            rtol, atol = reference_tolerances(dtype, accumulated=True)
            torch.testing.assert_close(xd.grad.cpu(), ref["dx"], rtol=rtol, atol=atol)
            torch.testing.assert_close(wd.grad.cpu(), ref["dw"], rtol=rtol, atol=atol)


# ---- scaled benchmark configurations, both kernel families -----------------------------------------
SCALED = [
    ("gpt2-small", dict(rows=640, hidden=768, vocab=5000)),
    ("llama3-8b", dict(rows=512, hidden=1024, vocab=6000)),
    ("large-vocab", dict(rows=384, hidden=576, vocab=9000)),
    ("14b-class", dict(rows=1024, hidden=640, vocab=2376)),
]


@pytest.mark.parametrize("force", ["tc", "tc1", "simt"])
@pytest.mark.parametrize("name,shape", SCALED, ids=[s[0] for s in SCALED])
def test_scaled_configurations(name, shape, force, monkeypatch):
    monkeypatch.setenv("HELION_B200_FORCE", force)
    cfg = inputs.scaled(inputs.CONFIGS[name], **shape)
    d = inputs.make_inputs(cfg)
    go = d["grad_out"] * (65536 / cfg.rows if name == "14b-class" else 1.0)
    _check(d["hidden"], d["weight"], d["target"], reduction=d["reduction"], grad_out=go)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 64, 65), (2, 8, 3), (127, 72, 129), (129, 136, 257), (130, 70, 300),
                                   (257, 200, 1000), (300, 768, 16064),
                                   (128, 512, 9000), (512, 1024, 20000),  # these two split the dX contraction
                                   (4096, 256, 65), (2048, 72, 130)])  # and these the dW contraction (char-LM heads)
def test_ragged_shapes(shape, dtype):
    n, h, v = shape
    g = torch.Generator().manual_seed(n * 7 + v)
    x = torch.randn(n, h, generator=g).to(dtype)
    w = (torch.randn(v, h, generator=g) / math.sqrt(h)).to(dtype)
    t = torch.randint(0, v, (n,), generator=g)
    _check(x, w, t, grad_out=torch.tensor(0.6))


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("force", ["tc", "simt"])
def test_reductions_ignore_index_and_upstream_gradient(reduction, force, monkeypatch):
    monkeypatch.setenv("HELION_B200_FORCE", force)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 150, 96, generator=g).bfloat16()
    w = (torch.randn(777, 96, generator=g) * 0.1).bfloat16()
    t = torch.randint(0, 777, (2, 150), generator=g)
    t[0, ::4] = -100
    go = torch.randn(2, 150, generator=g) if reduction == "none" else torch.tensor(65536.0)
    loss, _, _ = _check(x, w, t, reduction=reduction, grad_out=go)
    if reduction == "none":
        assert loss.shape == t.shape and float(loss.detach()[0, 0]) == 0.0
    _check(x, w, torch.where(t == -100, torch.full_like(t, 5), t), reduction=reduction, grad_out=go, ignore_index=5)


def test_int32_targets_and_inference_mode():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(64, 128, generator=g).bfloat16().to(DEV)
    w = torch.randn(500, 128, generator=g).bfloat16().to(DEV)
    t = torch.randint(0, 500, (64,), generator=g).to(DEV)
    a = ops.linear_cross_entropy(x, w, t)
    b = ops.linear_cross_entropy(x, w, t.int())
    assert torch.equal(a, b)
    with torch.inference_mode():
        c = ops.linear_cross_entropy(x.clone().requires_grad_(False), w, t)
    assert torch.equal(a, c) and not c.requires_grad


def test_empty_batch_and_single_row():
    w = torch.randn(300, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    x0 = torch.empty(0, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    t0 = torch.empty(0, dtype=torch.int64, device=DEV)
    loss = ops.linear_cross_entropy(x0, w, t0)
    assert float(loss) == 0.0  # reference: zero loss for no rows (tritium/ops/cross_entropy.py:578-581)
    dx, dw = ops.linear_cross_entropy_backward(torch.tensor(1.0, device=DEV), x0.detach(), w.detach(), t0,
                                               torch.empty(0, device=DEV))
    assert dx.shape == (0, 64) and float(dw.abs().sum()) == 0.0
    g = torch.Generator().manual_seed(8)
    _check(torch.randn(1, 64, generator=g).bfloat16(), torch.randn(300, 64, generator=g).bfloat16(), torch.tensor([7]))


def test_out_of_range_target_gives_infinite_loss_and_all_ignored_gives_nan():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(16, 64, generator=g).bfloat16().to(DEV)
    w = torch.randn(300, 64, generator=g).bfloat16().to(DEV)
    t = torch.randint(0, 300, (16,), generator=g).to(DEV)
    t[3] = 300  # matches no column and is not the ignored label: +inf, silently, like the reference
    assert math.isinf(float(ops.linear_cross_entropy(x, w, t)))
    all_ignored = torch.full((16,), -100, device=DEV)
    assert math.isnan(float(ops.linear_cross_entropy(x, w, all_ignored)))  # 0 / 0, as torch
    assert float(ops.linear_cross_entropy(x, w, all_ignored, reduction="sum")) == 0.0


def test_partial_needs_input_grad():
    g = torch.Generator().manual_seed(10)
    x = torch.randn(64, 128, generator=g).bfloat16().to(DEV)
    w = torch.randn(500, 128, generator=g).bfloat16().to(DEV)
    t = torch.randint(0, 500, (64,), generator=g).to(DEV)
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ops.linear_cross_entropy(xg, wg, t).backward()
    x1 = x.clone().requires_grad_(True)
    ops.linear_cross_entropy(x1, w, t).backward()
    w1 = w.clone().requires_grad_(True)
    ops.linear_cross_entropy(x, w1, t).backward()
    assert torch.equal(x1.grad, xg.grad) and torch.equal(w1.grad, wg.grad)


@pytest.mark.parametrize("force", ["tc", "tc1", "simt"])
def test_block_plans_agree_and_runs_are_bit_identical(force, monkeypatch):
    """Vocab bands, row chunks and the 2-D grid of blocks sum partial dX / dW in fp32 in a fixed order:
    every plan matches the single-block result to rounding, and the same plan twice is bit-identical."""
    monkeypatch.setenv("HELION_B200_FORCE", force)
    g = torch.Generator().manual_seed(12)
    x = torch.randn(1200, 256, generator=g).bfloat16()
    w = (torch.randn(2100, 256, generator=g) * 0.06).bfloat16()
    t = torch.randint(0, 2100, (1200,), generator=g)
    ref = oracle.expression(x, w, t)
    results = {}
    # 0: one block; 1.3 MB: vocab bands (dX summed); 1.1 MB after swapping roles: row chunks; 300 KB: 2-D
    for label, block, shape in [("single", 0, (1200, 2100)), ("bands", 1_300_000, (1200, 2100)),
                                ("chunks", 1_100_000, (2100, 1200)), ("grid", 300_000, (1200, 2100))]:
        monkeypatch.setenv("HELION_B200_BLOCK_BYTES", str(block))
        if shape == (1200, 2100):
            xx, ww, tt, rr = x, w, t, ref
        else:  # many more vocabulary rows than tokens favours row chunks
            xx, ww = w[:, :256].contiguous()[:2100], x[:1200].contiguous()
            tt = torch.randint(0, 1200, (2100,), generator=torch.Generator().manual_seed(13))
            rr = oracle.expression(xx, ww, tt)
        a = _run(xx, ww, tt)
        b = _run(xx, ww, tt)
        for u, v in zip(a, b):
            assert torch.equal(u, v), f"{label}: two runs differ"
        assert scaled_max_err(a[1], rr["dx"]) <= GRAD_RTOL_16BIT
        assert scaled_max_err(a[2], rr["dw"]) <= GRAD_RTOL_16BIT
        results[label] = a
    for label in ("bands", "grid"):
        assert scaled_max_err(results[label][1], results["single"][1].float()) <= 1e-2
        assert scaled_max_err(results[label][2], results["single"][2].float()) <= 1e-2


def test_both_kernel_families_agree():
    g = torch.Generator().manual_seed(14)
    x = torch.randn(300, 320, generator=g).half()
    w = (torch.randn(1500, 320, generator=g) * 0.05).half()
    t = torch.randint(0, 1500, (300,), generator=g)
    out = {}
    for force in ("tc", "simt"):
        os.environ["HELION_B200_FORCE"] = force
        out[force] = _run(x, w, t)
    os.environ.pop("HELION_B200_FORCE")
    assert rel_loss_err(out["tc"][0], out["simt"][0]) <= 1e-6
    assert scaled_max_err(out["tc"][1], out["simt"][1].float()) <= 4e-3
    assert scaled_max_err(out["tc"][2], out["simt"][2].float()) <= 4e-3


# ---- the GEMM core's operand layouts ---------------------------------------------------------------
@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("one_cta", [False, True], ids=["cta-pair", "one-cta"])
def test_gemm_core_operand_layouts(a_mn, b_mn, dtype, one_cta):
    g = torch.Generator().manual_seed(15)
    for m, n, k in [(128, 256, 64), (392, 520, 200), (136, 8, 72), (1304, 264, 136)]:
        a = torch.randn(m, k, generator=g).to(dtype)
        b = torch.randn(n, k, generator=g).to(dtype)
        ref = a.float() @ b.float().T
        out = ops.debug_gemm((a.T.contiguous() if a_mn else a).to(DEV), (b.T.contiguous() if b_mn else b).to(DEV), a_mn, b_mn,
                             one_cta=one_cta)
        assert scaled_max_err(out, ref) <= 1e-5


# ---- C ABI error paths ------------------------------------------------------------------------------
def test_c_abi_reports_small_workspace_and_forced_path_errors():
    L = _lib.lib()
    x = torch.randn(256, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(512, 64, device=DEV, dtype=torch.bfloat16)
    t = torch.randint(0, 512, (256,), device=DEV)
    stats = torch.empty(3, 256, device=DEV)
    ws = torch.empty(1024, dtype=torch.uint8, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    rc = L.lce_forward_stats(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, 256, 64, 512, 0, _lib.DTYPE_BF16,
                             stats.data_ptr(), ws.data_ptr(), ws.numel(), 0, s)
    assert rc == 3  # LCE_ERR_WS_TOO_SMALL
    big = torch.empty(1 << 22, dtype=torch.uint8, device=DEV)
    rc = L.lce_forward_stats(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, 256, 64, 512, 0, _lib.DTYPE_F32,
                             stats.data_ptr(), big.data_ptr(), big.numel(), _lib.FLAG_FORCE_TC, s)
    assert rc == 1  # fp32 has no tensor-core path here: an argument error, not a silent switch
    odd = torch.randn(256, 68, device=DEV, dtype=torch.bfloat16)  # 68 * 2 bytes is not a 16-byte pitch
    rc = L.lce_forward_stats(odd.data_ptr(), odd.data_ptr(), t.data_ptr(), 1, 256, 68, 256, 0, _lib.DTYPE_BF16,
                             stats.data_ptr(), big.data_ptr(), big.numel(), _lib.FLAG_FORCE_TC, s)
    assert rc == 2  # LCE_ERR_ALIGN


def test_vocab_shards_through_the_c_abi_merge_to_the_full_loss():
    """Four vocabulary shards computed one after the other on one GPU (what four ranks would compute),
    merged by lce_finalize: same loss as the unsharded call, and sharded dX partials sum to dX."""
    g = torch.Generator().manual_seed(16)
    x = torch.randn(200, 128, generator=g).bfloat16()
    w = (torch.randn(4 * 501, 128, generator=g) * 0.1).bfloat16()
    t = torch.randint(0, 4 * 501, (200,), generator=g)
    t[::11] = -100
    xd, wd, td = x.to(DEV), w.to(DEV), t.to(DEV)
    stats = torch.stack([ops.local_stats(xd, wd[r * 501:(r + 1) * 501].contiguous(), td, r * 501) for r in range(4)])
    loss, lse, count = ops.finalize(stats, td, "mean", -100, want_count=True)
    ref = oracle.expression(x, w, t)
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert int(count) == int((t != -100).sum())
    torch.testing.assert_close(lse.cpu(), ref["lse"], rtol=1e-4, atol=1e-4)
    dx_sum = torch.zeros(200, 128, device=DEV)
    for r in range(4):
        w_r = wd[r * 501:(r + 1) * 501].contiguous()
        dx_r, dw_r = ops._backward(torch.tensor(1.0, device=DEV), xd, w_r, td, lse, "mean", -100, None, r * 501,
                                   True, True)
        dx_sum += dx_r.float()
        assert scaled_max_err(dw_r, ref["dw"][r * 501:(r + 1) * 501]) <= GRAD_RTOL_16BIT
    assert scaled_max_err(dx_sum, ref["dx"]) <= GRAD_RTOL_16BIT


# ---- full-size checks -------------------------------------------------------------------------------
def test_gpt2_small_head_full_size_against_the_cpu_oracle():
    d = inputs.make_inputs(inputs.CONFIGS["gpt2-small"])
    ref = oracle.expression_chunked(d["hidden"], d["weight"], d["target"], chunk_rows=1024)
    loss, dx, dw = _run(d["hidden"], d["weight"], d["target"])
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert scaled_max_err(dx.view(4096, 768), ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_max_err(dw, ref["dw"]) <= GRAD_RTOL_16BIT


def test_llama3_head_full_size_properties_and_memory():
    """At the headline size the CPU oracle is out of reach; check the same expression evaluated in fp32
    on the GPU (TF32 off), gradient identities that need no oracle, and that no N x V buffer exists."""
    d = inputs.make_inputs(inputs.CONFIGS["llama3-8b"])
    n, h, v = 8192, 4096, 128256
    x = d["hidden"].to(DEV).requires_grad_(True)
    w = d["weight"].to(DEV).requires_grad_(True)
    t = d["target"].to(DEV)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    loss = ops.linear_cross_entropy(x, w, t)
    loss.backward()
    torch.cuda.synchronize()
    extra = torch.cuda.max_memory_allocated() - base
    grads = (n * h + v * h) * 2
    assert extra - grads < n * v * 2 // 3, "scratch must stay far below an N x V bf16 buffer"
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = oracle.expression_chunked(x.detach(), w.detach(), t, chunk_rows=512)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert scaled_max_err(x.grad.view(n, h), ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_max_err(w.grad, ref["dw"]) <= GRAD_RTOL_16BIT
    # size-independent identities: every row of G sums to zero, so dW summed over the vocabulary is zero
    # and ignored rows receive no gradient
    col_sum = w.grad.float().sum(dim=0)
    assert float(col_sum.abs().max()) <= 2e-2 * float(w.grad.float().abs().sum(dim=0).max())
    ignored = (t.view(-1) == -100)
    assert int(ignored.sum()) == 164 and float(x.grad.view(n, h)[ignored].abs().max()) == 0.0


def test_first_cuda_call_of_a_fresh_thread_may_be_this_library():
    """A thread that has made no CUDA runtime call yet (an autograd worker, a data-parallel thread) has no context
    bound; the tensor-map encoder is a driver call and needs one. The library binds it itself."""
    import threading

    g = torch.Generator().manual_seed(21)
    x = torch.randn(16, 512, generator=g).half().to(DEV)
    w = torch.randn(1024, 512, generator=g).half().to(DEV)
    t = torch.randint(0, 1024, (16,), generator=g).to(DEV)
    ref = ops.linear_cross_entropy(x, w, t)
    lse = torch.logsumexp(F.linear(x, w).float(), dim=-1)
    torch.cuda.synchronize()
    out = {}

    def work():
        try:
            loss = ops.linear_cross_entropy(x, w, t)
            dx, dw = ops.linear_cross_entropy_backward(torch.tensor(1.0, device=DEV), x, w, t, lse)
            torch.cuda.synchronize()
            out["ok"] = (float(loss), float(dx.float().abs().sum()), float(dw.float().abs().sum()))
        except Exception as exc:  # noqa: BLE001
            out["error"] = repr(exc)

    th = threading.Thread(target=work)
    th.start()
    th.join()
    assert "error" not in out, out
    assert abs(out["ok"][0] - float(ref)) <= 1e-6 * abs(float(ref))


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The op only enqueues work on the caller's stream (kernels and 4-byte memsets), so a forward + backward can
    be captured into a CUDA graph after a warm-up call and replayed on new data in the same buffers."""
    g = torch.Generator().manual_seed(22)
    n, h, v = 512, 256, 40000  # long enough for the dynamic tile deal (its counter memset is captured too)
    x = torch.randn(n, h, generator=g).bfloat16().to(DEV).requires_grad_(True)
    w = (torch.randn(v, h, generator=g) * 0.05).bfloat16().to(DEV).requires_grad_(True)
    t = torch.randint(0, v, (n,), generator=g).to(DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up outside the capture (allocations, attribute calls, tensor maps)
            x.grad = w.grad = None
            ops.linear_cross_entropy(x, w, t).backward()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    x.grad = w.grad = None
    with torch.cuda.graph(graph):
        loss = ops.linear_cross_entropy(x, w, t)
        loss.backward()
    with torch.no_grad():
        x.copy_(torch.randn(n, h, generator=g).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    ref = oracle.expression(x.detach().cpu(), w.detach().cpu(), t.cpu())
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert scaled_max_err(x.grad, ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_max_err(w.grad, ref["dw"]) <= GRAD_RTOL_16BIT


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_dx_reduce_scatter_emulated_on_one_gpu(world):
    """The vocabulary-parallel dX reduction, with the ranks played one after the other on ONE GPU (no kernel of
    the library waits on another rank, so the order does not matter): every rank's dX GEMM scatters its partial
    rows through the peer-store epilogue into the owners' staging buffers (here: local buffers), each owner sums
    its slice (`lce_dx_reduce_slice`) - and, the older form, sums and stores into every rank's final buffer
    (`lce_dx_reduce_gather`). Both must reproduce the unsharded dX; the local dW blocks the unsharded dW."""
    import ctypes

    L = _lib.lib()
    g = torch.Generator().manual_seed(30 + world)
    n, h, v = 1000, 256, world * 1002 + 5  # token count not a multiple of world * 128, uneven shards
    x = torch.randn(n, h, generator=g).bfloat16().to(DEV)
    w = (torch.randn(v, h, generator=g) * 0.08).bfloat16().to(DEV)
    t = torch.randint(0, v, (n,), generator=g).to(DEV)
    t[::13] = -100
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    loss = ops.linear_cross_entropy(xr, wr, t)
    loss.backward(torch.tensor(1.7, device=DEV))
    lse = torch.logsumexp(F.linear(x.float(), w.float()), dim=-1)
    go = torch.tensor(1.7, device=DEV)
    rpr = -(-n // world)
    staging = [torch.full((world, rpr, h), float("nan"), device=DEV) for _ in range(world)]
    code = _lib.DTYPE_BF16
    flags = _lib.FLAG_DX_F32
    from helion_b200 import parallel

    dws = []
    for r in range(world):
        start, end = parallel.shard_bounds(v, world, r)
        w_r = w[start:end].contiguous()
        dw_r = torch.empty_like(w_r)
        scatter = _lib.PeerScatter()
        for k in range(world):
            scatter.staging[k] = staging[k].data_ptr()
        scatter.rank, scatter.world = r, world
        ws = torch.empty(L.lce_backward_workspace_bytes(n, h, end - start, code, flags, 0), dtype=torch.uint8, device=DEV)
        _lib.check(L.lce_backward(x.data_ptr(), w_r.data_ptr(), t.data_ptr(), 1, lse.data_ptr(), go.data_ptr(), n, h,
                                  end - start, start, code, -100, _lib.REDUCTION_MEAN, None, dw_r.data_ptr(), ws.data_ptr(),
                                  ws.numel(), flags, 0, None, ctypes.byref(scatter), None,
                                  torch.cuda.current_stream().cuda_stream), "lce_backward")
        dws.append(dw_r)
    torch.cuda.synchronize()
    pieces = []
    finals = [torch.zeros(n, h, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    out_ptrs = (ctypes.c_void_p * world)(*[f.data_ptr() for f in finals])
    for r in range(world):
        piece = torch.zeros(rpr, h, dtype=torch.bfloat16, device=DEV)
        _lib.check(L.lce_dx_reduce_slice(staging[r].data_ptr(), world, r, n, h, code, piece.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream), "lce_dx_reduce_slice")
        _lib.check(L.lce_dx_reduce_gather(staging[r].data_ptr(), world, r, n, h, code, out_ptrs,
                                          torch.cuda.current_stream().cuda_stream), "lce_dx_reduce_gather")
        pieces.append(piece)
    torch.cuda.synchronize()
    dx = torch.cat(pieces)[:n]
    assert scaled_max_err(dx, xr.grad.float()) <= 8e-3
    assert all(torch.equal(f, dx) for f in finals)
    assert scaled_max_err(torch.cat(dws), wr.grad.float()) <= 8e-3
    assert _lib.device_status() == 0


@pytest.mark.parametrize("shape", [(16, 512, 1024), (128, 512, 1024), (128, 1024, 8192), (100, 264, 777), (1, 64, 300)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_very_small_problems_run_the_forward_in_one_launch(shape, reduction):
    """Few rows x few vocabulary tiles: the GEMM launch's last CTA merges the statistics and writes logsumexp and
    loss itself. One launch per forward, the oracle's loss, and the same bits call after call - more calls
    than the library has completion counters, so every counter is used again."""
    n, h, v = shape
    g = torch.Generator().manual_seed(n + h + v)
    x = torch.randn(n, h, generator=g).to(torch.float16).to(DEV)
    w = (torch.randn(v, h, generator=g) / h ** 0.5).to(torch.float16).to(DEV)
    t = torch.randint(0, v, (n,), generator=g)
    if n > 4:
        t[::5] = -100
    t = t.to(DEV)
    L = _lib.lib()
    first = ops.linear_cross_entropy(x, w, t, reduction=reduction)
    torch.cuda.synchronize()
    before = L.lce_launch_count()
    again = ops.linear_cross_entropy(x, w, t, reduction=reduction)
    torch.cuda.synchronize()
    assert L.lce_launch_count() - before == 1
    assert torch.equal(first, again)
    ref = F.cross_entropy(F.linear(x.float(), w.float()), t, reduction=reduction)
    torch.testing.assert_close(first.float(), ref, rtol=2e-3, atol=2e-3)
    if reduction == "mean" and shape == (16, 512, 1024):
        for _ in range(4200):
            again = ops.linear_cross_entropy(x, w, t, reduction=reduction)
        assert torch.equal(first, again)
        assert _lib.device_status() == 0


@pytest.mark.parametrize("shape", [(16, 512, 1024), (128, 1024, 8192), (100, 264, 777), (1, 64, 300)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_backward_of_a_handful_of_tokens_computes_dx_and_dw_in_one_launch(shape, dtype):
    """At most 128 tokens: the recompute launch, then ONE launch that carries both gradient products (plus a sum
    pass where the long vocabulary contraction of dX was cut into slices). Gradients against autograd of the
    fp32 expression, and the same bits on a second run."""
    n, h, v = shape
    g = torch.Generator().manual_seed(7 * n + h + v)
    x = torch.randn(n, h, generator=g).to(dtype).to(DEV)
    w = (torch.randn(v, h, generator=g) / h ** 0.5).to(dtype).to(DEV)
    t = torch.randint(0, v, (n,), generator=g)
    if n > 4:
        t[::7] = -100
    t = t.to(DEV)
    go = torch.tensor(0.75, device=DEV)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    z = F.linear(xr, wr)
    (F.cross_entropy(z, t) * go).backward()
    lse = torch.logsumexp(z.detach(), dim=-1)
    L = _lib.lib()
    dx, dw = ops.linear_cross_entropy_backward(go, x, w, t, lse)
    torch.cuda.synchronize()
    before = L.lce_launch_count()
    dx2, dw2 = ops.linear_cross_entropy_backward(go, x, w, t, lse)
    torch.cuda.synchronize()
    assert L.lce_launch_count() - before in (2, 3)  # recompute + both products (+ the slice sum of dX)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)
    assert scaled_max_err(dx, xr.grad) <= GRAD_RTOL_16BIT and scaled_max_err(dw, wr.grad) <= GRAD_RTOL_16BIT
    assert _lib.device_status() == 0
