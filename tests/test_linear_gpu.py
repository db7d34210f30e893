"""Sharded F.linear on the tcgen05 path against the CPU oracle (float64 contraction of the same
bf16 inputs).  bf16 tolerance from the north star: 1e-2 relative (plus 1e-2 of the output's RMS
for entries near zero).  Shapes are the per-rank shard shapes of the benchmark configurations."""
import pytest
import torch

import hap_b200
from hap_b200 import linear_ops as L
from oracle import linear_math as lm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gen(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def close(got, want, what=""):
    got = got.detach().double().cpu()
    rms = float(want.pow(2).mean().sqrt())
    err = (got - want).abs()
    bound = 1e-2 * want.abs() + 1e-2 * rms
    bad = int((err > bound).sum())
    assert bad == 0, f"{what}: {bad} of {want.numel()} entries off, max err {float(err.max()):.4g}, rms {rms:.4g}"


FWD_SHAPES = [  # (m, n, k)
    (38, 4096, 1024), (26, 4096, 1024), (38, 1024, 4096),      # MLP config, data parallel, ratios [.6,.4]
    (64, 2458, 1024), (64, 1638, 1024), (64, 614, 4096),       # MLP config, column parallel shards (n % 8 != 0)
    (300, 520, 72), (1, 8, 8), (129, 257, 136),                # ragged tiles, k tail
    (1000, 768, 3072), (2048, 2304, 768),                      # transformer projections
    (513, 154, 768),                                           # r8 tail shard of a 3072-wide FFN
]


@pytest.mark.parametrize("m,n,k", FWD_SHAPES)
def test_forward_matches_oracle(m, n, k):
    x, w, b = gen((m, k), 1), gen((n, k), 2, k ** -0.5), gen((n,), 3)
    want = lm.linear_forward(x, w, b)
    got = L.linear_forward(x.to(DEV), w.to(DEV), b.to(DEV))
    L.gemm_status()
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    close(got, want, "forward")
    got32 = L.linear_forward(x.to(DEV), w.to(DEV), None, out_dtype=torch.float32)
    L.gemm_status()
    close(got32, lm.linear_forward(x, w, None), "forward fp32 out")


@pytest.mark.parametrize("act", ["relu", "gelu", "sigmoid"])
def test_fused_epilogues(act):
    m, n, k = 200, 384, 256
    x, w, b = gen((m, k), 4), gen((n, k), 5, k ** -0.5), gen((n,), 6)
    got = L.linear_forward(x.to(DEV), w.to(DEV), b.to(DEV), epilogue=act)
    L.gemm_status()
    close(got, lm.linear_forward(x, w, b, act), act)


BWD_SHAPES = [(38, 4096, 1024), (26, 1024, 4096), (300, 520, 72), (1000, 768, 3072), (2048, 2304, 768), (8, 8, 8),
              (77, 1000, 768), (4096, 768, 768), (8192, 256, 520),      # the last ones take the split-K path in wgrad
              (64, 2458, 1024), (64, 410, 4096)]                       # column-parallel shards, width not a multiple of 8


@pytest.mark.parametrize("m,n,k", BWD_SHAPES)
def test_backward_matches_oracle(m, n, k):
    x, w, b = gen((m, k), 7), gen((n, k), 8, k ** -0.5), gen((n,), 9)
    g = gen((m, n), 10)
    xd, wd, bd = (t.to(DEV).requires_grad_(True) for t in (x, w, b))
    y = hap_b200.linear(xd, wd, bd)
    y.backward(g.to(DEV))
    L.gemm_status()
    dx, dw, db = lm.linear_backward(g, x, w)
    close(xd.grad, dx, "dgrad")
    close(wd.grad, dw, "wgrad")
    close(bd.grad, db, "bias grad")


# The per-GPU GEMMs of the Transformer-LM configuration at full size (8192 tokens): too large for a
# full float64 product on the CPU in seconds, so the oracle is evaluated on a seeded sample of rows
# and columns of each result (the whole contraction length for every sampled entry).
FULL_SHAPES = [(8192, 33280, 768),     # vocabulary projection: its input gradient takes the 520-slice split-K path
               (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072), (8192, 2304, 768)]


def _sample(extent, count, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(extent, generator=g)[:min(count, extent)].sort().values
    # always include the edges of the first / last tile
    return torch.unique(torch.cat([idx, torch.tensor([0, extent - 1, min(extent - 1, 255), min(extent - 1, 256)])]))


@pytest.mark.parametrize("m,n,k", FULL_SHAPES)
def test_full_size_lm_gemms_on_sampled_entries(m, n, k):
    x, w, b = gen((m, k), 21), gen((n, k), 22, k ** -0.5), gen((n,), 23)
    g = gen((m, n), 24)
    xd, wd, bd = (t.to(DEV).requires_grad_(True) for t in (x, w, b))
    y = hap_b200.linear(xd, wd, bd)
    y.backward(g.to(DEV))
    L.gemm_status()
    rows, cols, ks = _sample(m, 192, 31), _sample(n, 384, 32), _sample(k, 256, 33)
    xs, ws = x.double(), w.double()
    g_rows, g_cols = g[rows].double(), g[:, cols].double()     # slices first: the full matrix in float64 is 2 GB
    # forward: y[rows, cols]
    want = xs[rows] @ ws[cols].t() + b.double()[cols]
    close(y.detach()[rows.to(DEV)][:, cols.to(DEV)], want, "forward (sampled)")
    # dgrad: dx[rows, ks] = g[rows, :] @ w[:, ks]
    want = g_rows @ ws[:, ks]
    close(xd.grad[rows.to(DEV)][:, ks.to(DEV)], want, "dgrad (sampled)")
    # wgrad: dw[cols, ks] = g[:, cols]^T @ x[:, ks]
    want = g_cols.t() @ xs[:, ks]
    close(wd.grad[cols.to(DEV)][:, ks.to(DEV)], want, "wgrad (sampled)")
    close(bd.grad[cols.to(DEV)], g_cols.sum(0), "bias grad (sampled)")


def test_leading_dims_are_flattened():
    x, w = gen((4, 50, 64), 11), gen((96, 64), 12)
    xd, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    y = hap_b200.linear(xd, wd)
    assert y.shape == (4, 50, 96)
    y.sum().backward()
    L.gemm_status()
    close(y, lm.linear_forward(x.reshape(-1, 64), w).reshape(4, 50, 96))
    dx, dw, _ = lm.linear_backward(torch.ones(4, 50, 96), x, w)
    close(xd.grad, dx)
    close(wd.grad, dw)


FP32_SHAPES = [(38, 4096, 1024), (26, 1024, 4096), (64, 2458, 1024), (64, 410, 4096), (7, 5, 3), (130, 67, 33)]


@pytest.mark.parametrize("m,n,k", FP32_SHAPES)
def test_fp32_forward_and_backward_within_1e5(m, n, k):
    """The fp32 configuration (2-layer MLP, ratios [.6,.4]) must match to 1e-5 relative."""
    g = torch.Generator().manual_seed(39)
    x, w, b = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g) * k ** -0.5, torch.randn(n, generator=g)
    gy = torch.randn(m, n, generator=g)
    xd, wd, bd = (t.to(DEV).requires_grad_(True) for t in (x, w, b))
    y = hap_b200.linear(xd, wd, bd)
    y.backward(gy.to(DEV))
    assert y.dtype == torch.float32
    dx, dw, db = lm.linear_backward(gy, x, w)
    for got, want in ((y, lm.linear_forward(x, w, b)), (xd.grad, dx), (wd.grad, dw), (bd.grad, db)):
        rms = float(want.pow(2).mean().sqrt())
        err = (got.detach().double().cpu() - want).abs()
        assert float((err - 1e-5 * want.abs()).max()) <= 1e-5 * rms


def test_unsupported_inputs_raise():
    x, w = gen((8, 12), 1).to(DEV), gen((8, 12), 2).to(DEV)
    with pytest.raises(ValueError):
        L.linear_forward(x, w, None)                       # bf16 with k % 8 != 0
    with pytest.raises(TypeError):
        L.linear_forward(x.half(), w.half(), None)
    with pytest.raises(TypeError):
        L.linear_forward(x.float(), w, None)                # mixed dtypes
    with pytest.raises(RuntimeError):
        L.linear_forward(x.cpu(), w.cpu(), None)
