"""The batch-norm kernels behind ``cudnn_batch_norm`` / ``cudnn_batch_norm_backward`` against
the float64 oracle (GPU)."""
import pytest
import torch

import actnn_oracle as O

pytestmark = pytest.mark.gpu

# tolerance: outputs are rounded once to the tensor dtype from float32 arithmetic
TOL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}

SHAPES = [
    (8, 64, 56, 56),     # 16-byte vectors, several splits per channel
    (16, 32, 14, 14),    # 196 positions: 8-byte vectors for 16-bit types
    (16, 48, 7, 7),      # 49 positions: scalar path
    (3, 5, 6, 10),       # ragged everything
    (64, 10),            # [N, C]
    (4, 6, 33),          # [N, C, L]
    (1, 8, 16, 16),      # one sample
    (32, 300, 4, 4),     # more channels than blocks wanted: one split
]


def _inputs(shape, dtype, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    C = shape[1]
    x = (torch.randn(shape, generator=g) * 1.7 + torch.linspace(-3, 3, C).view([1, C] + [1] * (len(shape) - 2)))
    gy = torch.randn(shape, generator=g)
    w, b = torch.randn(C, generator=g), torch.randn(C, generator=g)
    rm, rv = torch.randn(C, generator=g), torch.rand(C, generator=g) + 0.5
    return x.to(dtype).to(dev), gy.to(dtype).to(dev), w.to(dev), b.to(dev), rm.to(dev), rv.to(dev)


def _close(got, want, tol):
    want = want.to(got.device)
    scale = max(1.0, float(want.abs().max()))
    return float((got.double() - want.double()).abs().max()) <= tol * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_batch_norm_forward_backward(cuda_device, shape, dtype):
    from actnn_b200.cpp_extension import backward_func as bf
    x, gy, w, b, rm, rv = _inputs(shape, dtype, cuda_device)
    rm0, rv0 = rm.clone(), rv.clone()
    y, mean, invstd, reserve = bf.cudnn_batch_norm(x, w, b, rm, rv, True, 0.1, 1e-5)
    y_o, mean_o, invstd_o, rm_o, rv_o = O.batch_norm_forward(x.cpu(), w.cpu(), b.cpu(), rm0.cpu(), rv0.cpu(), 0.1, 1e-5)
    tol = TOL[dtype]
    assert y.dtype == dtype and y.shape == x.shape and reserve.numel() == 0
    assert _close(y, y_o, tol)
    assert _close(mean, mean_o, 1e-5) and _close(invstd, invstd_o, 1e-4)
    assert _close(rm, rm_o, 1e-5) and _close(rv, rv_o, 1e-5)
    dx, dw, db = bf.cudnn_batch_norm_backward(x, gy, w, rm, rv, mean, invstd, 1e-5, reserve)
    dx_o, dw_o, db_o = O.batch_norm_backward(x.cpu(), gy.cpu(), w.cpu(), mean.cpu(), invstd.cpu())
    assert dx.dtype == dtype and _close(dx, dx_o, tol)
    assert _close(dw, dw_o, 1e-4) and _close(db, db_o, 1e-4)


def test_batch_norm_matches_cudnn_and_is_deterministic(cuda_device):
    """Against the operator the reference calls, and bit-equal on a second run."""
    from actnn_b200.cpp_extension import backward_func as bf
    x, gy, w, b, rm, rv = _inputs((32, 64, 28, 28), torch.float16, cuda_device, seed=3)
    rm_t, rv_t = rm.clone(), rv.clone()
    y_t, mean_t, invstd_t, res_t = torch.ops.aten.cudnn_batch_norm(x, w, b, rm_t, rv_t, True, 0.1, 1e-5)
    dx_t, dw_t, db_t = torch.ops.aten.cudnn_batch_norm_backward(x, gy, w, rm_t, rv_t, mean_t, invstd_t, 1e-5, res_t)
    rm1, rv1 = rm.clone(), rv.clone()
    y, mean, invstd, res = bf.cudnn_batch_norm(x, w, b, rm1, rv1, True, 0.1, 1e-5)
    dx, dw, db = bf.cudnn_batch_norm_backward(x, gy, w, rm1, rv1, mean, invstd, 1e-5, res)
    assert _close(y, y_t, 2e-3) and _close(dx, dx_t, 2e-3)
    assert _close(mean, mean_t, 1e-5) and _close(invstd, invstd_t, 1e-4)
    assert _close(rm1, rm_t, 1e-5) and _close(rv1, rv_t, 1e-5)
    assert _close(dw, dw_t, 2e-4) and _close(db, db_t, 2e-4)
    rm2, rv2 = rm.clone(), rv.clone()
    y2, mean2, invstd2, _ = bf.cudnn_batch_norm(x, w, b, rm2, rv2, True, 0.1, 1e-5)
    dx2, dw2, db2 = bf.cudnn_batch_norm_backward(x, gy, w, rm2, rv2, mean2, invstd2, 1e-5, res)
    for a, c in ((y, y2), (mean, mean2), (invstd, invstd2), (dx, dx2), (dw, dw2), (db, db2), (rm1, rm2)):
        assert torch.equal(a, c)


def test_batch_norm_large_offset_variance(cuda_device):
    """A mean far above the deviation: the shifted sums keep the variance."""
    from actnn_b200.cpp_extension import backward_func as bf
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(16, 8, 32, 32, generator=g) * 0.01 + 100.0).to(cuda_device)
    y, mean, invstd, _ = bf.cudnn_batch_norm(x, None, None, None, None, True, 0.1, 1e-5)
    _, mean_o, invstd_o, _, _ = O.batch_norm_forward(x.cpu(), None, None, None, None, 0.1, 1e-5)
    assert _close(invstd, invstd_o, 1e-3) and _close(mean, mean_o, 1e-6)


@pytest.fixture()
def actnn(cuda_device):
    import actnn_b200
    from actnn_b200.conf import QuantizationConfig
    fresh = QuantizationConfig()
    actnn_b200.config.__dict__.update(fresh.__dict__)
    yield actnn_b200
    actnn_b200.config.__dict__.update(fresh.__dict__)


def test_batch_norm_module_trains_like_torch(actnn, cuda_device):
    """QBatchNorm2d at level L0 (no compression) against nn.BatchNorm2d."""
    actnn.set_optimization_level("L0")
    torch.manual_seed(0)
    ref = torch.nn.BatchNorm2d(24).to(cuda_device)
    ours = actnn.QBatchNorm2d(24).to(cuda_device)
    ours.load_state_dict(ref.state_dict())
    x = torch.randn(8, 24, 12, 12, device=cuda_device)
    xr, xo = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    yr, yo = ref(xr), ours(xo)
    gy = torch.randn_like(yr)
    yr.backward(gy)
    yo.backward(gy)
    assert torch.allclose(yo, yr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(xo.grad, xr.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ours.weight.grad, ref.weight.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(ours.bias.grad, ref.bias.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(ours.running_var, ref.running_var, rtol=1e-5, atol=1e-6)
    assert torch.allclose(ours.running_mean, ref.running_mean, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(8, 32, 14, 14), (6, 10, 7, 7), (16, 24)])
def test_sync_halves_match_the_aten_operators(cuda_device, shape, dtype):
    """batch_norm_stats / elemt / backward_reduce / backward_elemt against the ATen operators
    of the same names (the ones the reference's synchronised batch norm calls)."""
    from actnn_b200.cpp_extension import backward_func as bf
    x, gy, w, b, _, _ = _inputs(shape, dtype, cuda_device, seed=9)
    tol = TOL[dtype]
    mean, invstd = bf.batch_norm_stats(x, 1e-5)
    mean_t, invstd_t = torch.batch_norm_stats(x, 1e-5)
    assert _close(mean, mean_t, 1e-5) and _close(invstd, invstd_t, 1e-4)
    y = bf.batch_norm_elemt(x, w, b, mean_t, invstd_t, 1e-5)
    assert _close(y, torch.batch_norm_elemt(x, w, b, mean_t, invstd_t, 1e-5), tol)
    sum_dy, sum_dy_xmu, gw, gb = bf.batch_norm_backward_reduce(gy, x, mean_t, invstd_t, w, True, True, True)
    sum_dy_t, sum_dy_xmu_t, gw_t, gb_t = torch.batch_norm_backward_reduce(gy, x, mean_t, invstd_t, w, True, True, True)
    # the sums themselves are checked in float64 (ATen's own float16 sums are off by ~3e-4)
    dims = [d for d in range(x.dim()) if d != 1]
    view = [1, -1] + [1] * (x.dim() - 2)
    sum_dy_64 = gy.double().sum(dim=dims)
    sum_dy_xmu_64 = (gy.double() * (x.double() - mean_t.double().view(view))).sum(dim=dims)
    assert _close(sum_dy, sum_dy_64, 2e-5) and _close(sum_dy_xmu, sum_dy_xmu_64, 2e-5)
    assert _close(gw, sum_dy_xmu_64 * invstd_t.double(), 2e-5) and _close(gb, sum_dy_64, 2e-5)
    assert _close(sum_dy, sum_dy_t, 2e-3) and _close(gw, gw_t, 2e-3)
    # two "ranks" with the same batch: sums and counts double
    per_rank = x.numel() // x.shape[1]
    count = torch.tensor([per_rank, per_rank], dtype=torch.float32, device=cuda_device)
    dx = bf.batch_norm_backward_elemt(gy, x, mean_t, invstd_t, w, 2 * sum_dy_t, 2 * sum_dy_xmu_t, count)
    dx_t = torch.batch_norm_backward_elemt(gy, x, mean_t, invstd_t, w, 2 * sum_dy_t, 2 * sum_dy_xmu_t, count.int())
    assert _close(dx, dx_t, tol)


def test_sync_batch_norm_op_in_a_one_rank_group_matches_batch_norm(actnn, cuda_device):
    """ops.sync_batch_norm itself (all_gather / all_reduce over a one-rank NCCL group) against
    nn.BatchNorm2d."""
    import os
    import torch.distributed as dist
    from actnn_b200 import ops
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=cuda_device)
    try:
        actnn.set_optimization_level("L0")
        torch.manual_seed(1)
        ref = torch.nn.BatchNorm2d(12).to(cuda_device)
        w = ref.weight.detach().clone().requires_grad_(True)
        b = ref.bias.detach().clone().requires_grad_(True)
        rm, rv = ref.running_mean.clone(), ref.running_var.clone()
        x = torch.randn(6, 12, 9, 9, device=cuda_device)
        xr, xo = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        yr = ref(xr)
        yo = ops.sync_batch_norm.apply(xo, w, b, rm, rv, ref.eps, ref.momentum, dist.group.WORLD, 1, None)
        gy = torch.randn_like(yr)
        yr.backward(gy)
        yo.backward(gy)
        assert torch.allclose(yo, yr, rtol=1e-4, atol=1e-5)
        assert torch.allclose(xo.grad, xr.grad, rtol=1e-4, atol=1e-5)
        assert torch.allclose(w.grad, ref.weight.grad, rtol=1e-4, atol=1e-4)
        assert torch.allclose(b.grad, ref.bias.grad, rtol=1e-4, atol=1e-4)
        assert torch.allclose(rv, ref.running_var, rtol=1e-5, atol=1e-6)
        assert torch.allclose(rm, ref.running_mean, rtol=1e-5, atol=1e-6)
    finally:
        if created:
            dist.destroy_process_group()


def test_resnet18_trains_like_stock_torch_at_level_L0(actnn, cuda_device):
    """A ResNet-18 through QModule without compression (level L0: only the batch-norm, ReLU and
    max-pool kernels differ from stock torch) against the stock model: same logits, gradients
    equal to within what a 1e-7 perturbation of the input does to the stock model itself
    (a randomly initialised 18-layer net with batch 16 amplifies rounding differences to
    ~1e-2 in the gradients), and the same losses over three SGD steps."""
    import copy
    import torchvision
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    try:
        actnn.set_optimization_level("L0")
        torch.manual_seed(0)
        stock = torchvision.models.resnet18(num_classes=10).to(cuda_device).train()
        ours = actnn.QModule(copy.deepcopy(stock)).train()
        x = torch.randn(16, 3, 64, 64, device=cuda_device)
        y = torch.randint(0, 10, (16,), device=cuda_device)
        out_s, out_o = stock(x), ours(x)
        assert torch.allclose(out_o, out_s, rtol=1e-3, atol=1e-3)
        torch.nn.functional.cross_entropy(out_s, y).backward()
        torch.nn.functional.cross_entropy(out_o, y).backward()
        for (name, p), q in zip(stock.named_parameters(), ours.model.parameters()):
            assert float((p.grad - q.grad).norm()) <= 5e-2 * float(p.grad.norm()) + 1e-6, name
        losses = []
        for model in (stock, ours):
            opt = torch.optim.SGD(model.parameters(), lr=0.01)
            trace = []
            for _ in range(3):
                opt.zero_grad(set_to_none=True)
                loss = torch.nn.functional.cross_entropy(model(x), y)
                loss.backward()
                opt.step()
                trace.append(float(loss.detach()))
            losses.append(trace)
        assert all(abs(a - b) <= 2e-2 * max(1.0, abs(a)) for a, b in zip(*losses)), losses
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32


# ------------------------------------------------------------------------------ statistics + min / max in one read
FUSED_SHAPES = [
    (8, 64, 56, 56),      # HW = 3136: tasks of 8 rows, two channels per task at most
    (4, 256, 28, 28),     # HW = 784: tasks of 3 rows, most groups straddle two channels
    (3, 16, 16, 16),      # HW = 256: one row per task, a group is exactly a channel plane
    (2, 6, 32, 40),       # HW = 1280, ragged last task of every sample
    (5, 64, 112, 112),    # the stem of a ResNet
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", FUSED_SHAPES)
def test_statistics_and_group_minmax_from_one_read(cuda_device, shape, dtype):
    """``batch_norm_stats_minimax``: min / max of every 256-group exactly as the minimax kernel
    (and ``torch.min/max``) gives them, statistics and running statistics as the plain batch-norm
    kernels / ``torch.batch_norm_stats`` give them."""
    from actnn_b200.cpp_extension import backward_func as bf
    x, _, w, b, rm, rv = _inputs(shape, dtype, cuda_device, seed=3)
    rm_ref, rv_ref = rm.clone(), rv.clone()
    got = bf.batch_norm_stats_minimax(x, w, b, rm, rv, 0.1, 1e-5)
    assert got is not None
    mn, mx, mean, invstd = got
    groups = x.reshape(shape[0], -1, 256)
    assert torch.equal(mn.view(shape[0], -1), groups.min(dim=2)[0])
    assert torch.equal(mx.view(shape[0], -1), groups.max(dim=2)[0])
    mean_t, invstd_t = torch.batch_norm_stats(x.float(), 1e-5)
    assert _close(mean, mean_t, 2e-5) and _close(invstd, invstd_t, 2e-4)
    # running statistics: the same update the unfused kernel makes
    _, save_mean, save_invstd, _ = bf.cudnn_batch_norm(x, w, b, rm_ref, rv_ref, True, 0.1, 1e-5)
    assert _close(mean, save_mean, 1e-5) and _close(invstd, save_invstd, 1e-4)
    assert _close(rm, rm_ref, 1e-5) and _close(rv, rv_ref, 1e-4)
    # bit-reproducible
    mn2, mx2, mean2, invstd2 = bf.batch_norm_stats_minimax(x, w, b, None, None, 0.1, 1e-5)
    assert torch.equal(mean2, mean) and torch.equal(invstd2, invstd) and torch.equal(mn2, mn)


def test_statistics_and_minmax_pass_declines_other_geometries(cuda_device):
    from actnn_b200.cpp_extension import backward_func as bf
    for shape in ((16, 32, 14, 14), (16, 48, 7, 7), (4, 3, 16, 24), (64, 10)):
        x = torch.randn(shape, device=cuda_device)
        assert bf.batch_norm_stats_minimax(x, None, None, None, None, 0.1, 1e-5) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_quantized_batch_norm_takes_the_one_read_path_and_matches_the_two_read_path(actnn, cuda_device, dtype):
    """ops.batch_norm at level L3 on a covered geometry: output, gradients and the saved
    compressed activation are the same as with the separate minimax and statistics passes."""
    from actnn_b200 import ops
    from actnn_b200.cpp_extension import backward_func as bf
    actnn.set_optimization_level("L3")
    N, C, H, W = 6, 32, 16, 24
    x, gy, w, b, rm, rv = _inputs((N, C, H, W), dtype, cuda_device, seed=5)
    gen = torch.cuda.default_generators[cuda_device.index or 0]
    results = []
    for fused in (True, False):
        scheme = actnn.QBNScheme()
        real = bf.batch_norm_stats_minimax
        calls = []
        if fused:
            bf.batch_norm_stats_minimax = lambda *a, **k: (calls.append(1), real(*a, **k))[1]
        else:
            bf.batch_norm_stats_minimax = lambda *a, **k: None
        try:
            gen.manual_seed(77)
            xi = x.clone().requires_grad_(True)
            wi, bi = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
            rmi, rvi = rm.clone(), rv.clone()
            y = ops.batch_norm.apply(xi, rmi, rvi, wi, bi, True, 0.1, 1e-5, scheme)
            y.backward(gy)
        finally:
            bf.batch_norm_stats_minimax = real
        assert bool(calls) == fused
        results.append((y.detach(), xi.grad, wi.grad, bi.grad, rmi, rvi))
    tol = TOL[dtype]
    for a, r in zip(*results):
        assert _close(a, r, 4 * tol)
    ref = torch.nn.functional.batch_norm(x.float(), rm.clone(), rv.clone(), w, b, True, 0.1, 1e-5)
    assert _close(results[0][0].float(), ref, 4 * tol)
